"""GPU tests of the Ramopel path: the engine (scheduler, paged latent cache, recurrent-state slots, kernels)
against oracle/ramopel.py — a plain fp64 restatement that recomputes every position from the tokens, with no
cache and no batching.  The configurations are small, differ from one another in every size, and are drawn
here; the fp32 engine is held to a tight bound, the bf16 engine to a rounding-sized one."""
import ctypes as C
import json
import os

import numpy as np
import pytest
import torch

from oracle import ramopel as O
from tests.ramopel_util import DENSE, MOE, MOE_PLAIN, attn, checkpoint, delta, rel_err, small_spec, tokens

pytestmark = pytest.mark.gpu
F32_TOL, BF16_TOL = 2e-4, 6e-2


def build(spec, sd, dtype=torch.float32, max_tokens=512, max_seqs=4, num_blocks=None):
    from llmq_b200.model import BLOCK_SIZE, Engine, NativeModel
    from llmq_b200.ramopel import engine_weights

    nb = num_blocks or (max_tokens // BLOCK_SIZE + max_seqs)
    model = NativeModel(spec, engine_weights(spec, sd), max_tokens=max_tokens, max_seqs=max_seqs,
                        max_model_len=max_tokens, num_blocks=nb, dtype=dtype, max_logit_rows=max_tokens)
    eng = Engine(model, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens, max_model_len=model.max_model_len)
    return model, eng


def oracle_logits(spec, sd, toks):
    return O.forward(spec.to_config(), sd, toks, torch.float64).numpy()


def replay_cut(eng, rid, toks, cuts):
    """feed toks to request rid in portions of the given sizes (the rest one by one); logits of every place"""
    out, at, cuts = [], 0, list(cuts)
    while at < len(toks):
        n = min(cuts.pop(0) if cuts else 1, len(toks) - at)
        out.append(eng.step_replay([(rid, toks[at:at + n], list(range(n)))]))
        at += n
    return np.concatenate(out)


# ---- every mechanism alone: a one-layer model around it --------------------------------------------------
ONE_LAYER = {
    "latent_attention": [attn()],
    "latent_attention_wide": [attn(heads=11, dim=24, rot_dim=4, vdim=8, q_rank=16, kv_rank=72, window=5)],
    "latent_attention_all_keys": [attn(window=0)],
    "latent_attention_borrowed": [attn(), attn(heads=4, dim=8, vdim=8, window=3, kv_from=0)],
    "general_delta": [delta()],
    "general_delta_odd": [delta(heads=5, dim=24, rank=3)],
    "polynorm": [delta(heads=1, dim=32, **DENSE)],
    "experts_shared": [delta(heads=1, dim=32, **MOE)],
    "experts_top1": [delta(heads=1, dim=32, **MOE_PLAIN)],
    "experts_all_chosen": [delta(heads=1, dim=32, ff="moe", ff_dim=16, n_experts=3, top_k=3, expert_limit=0.5)],
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mechanism_alone(cuda, name, dtype):
    spec = small_spec(width=80, vocab=97, layers=ONE_LAYER[name])
    sd = checkpoint(spec, seed=11)
    toks = tokens(45, spec.vocab, 5)
    model, eng = build(spec, sd, dtype)
    tap = torch.zeros(spec.n_layers, len(toks), spec.width, device=cuda)
    model.set_layer_tap(tap)
    got = eng.step_replay([(1, toks, list(range(len(toks))))])
    model.set_layer_tap(None)
    want, stream = O.forward(spec.to_config(), sd, toks, torch.float64, keep_layers=True)
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    assert rel_err(tap.cpu().numpy()[-1], stream[-1].numpy()) < tol, name
    assert rel_err(got, want.numpy()) < tol, name
    eng.close()
    model.close()


def _ops():
    from llmq_b200 import lib as L
    return L, L.load()


@pytest.mark.parametrize("rows,F", [(1, 7), (33, 320), (5, 1000)])
def test_polynorm_op(cuda, rows, F):
    L, lib = _ops()
    g = torch.Generator().manual_seed(1)
    z = torch.randn(rows, F, generator=g) * 2
    coef = torch.tensor([0.7, -0.3, 0.2, 0.1])
    y = torch.empty(rows, F, device=cuda)
    zd, cd = z.to(cuda), coef.to(cuda)
    L.check(lib.b200q_polynorm(zd.data_ptr(), cd.data_ptr(), y.data_ptr(), rows, F, 1e-5, L.DTYPE_F32, None))
    torch.cuda.synchronize()
    zz = z.double()
    want = (0.7 * O.rms_unit(zz, 1e-5) - 0.3 * O.rms_unit(zz * zz, 1e-5) + 0.2 * O.rms_unit(zz ** 3, 1e-5) + 0.1)
    assert rel_err(y.cpu().numpy(), want.numpy()) < 1e-5


def test_router_op_ties_and_softmax(cuda):
    L, lib = _ops()
    T_, E, top = 9, 7, 3
    z = torch.randn(T_, E, generator=torch.Generator().manual_seed(2))
    z[0] = torch.tensor([1.0, 5.0, 5.0, -1.0, 5.0, 0.0, 2.0])    # ties: the lowest indices win
    zc = z.to(cuda)
    idx = torch.zeros(T_, top, dtype=torch.int32, device=cuda)
    wts = torch.zeros(T_, top, device=cuda)
    goff = torch.zeros(E + 1, dtype=torch.int32, device=cuda)
    perm = torch.zeros(T_ * top, dtype=torch.int32, device=cuda)
    ppos = torch.zeros(T_ * top, dtype=torch.int32, device=cuda)
    tab = torch.zeros(T_ * top // 128 + E + 1, 4, dtype=torch.int32, device=cuda)
    ntl = torch.zeros(1, dtype=torch.int32, device=cuda)
    L.check(lib.b200q_moe_route(zc.data_ptr(), T_, E, top, idx.data_ptr(), wts.data_ptr(), goff.data_ptr(),
                                perm.data_ptr(), ppos.data_ptr(), tab.data_ptr(), ntl.data_ptr(), None))
    torch.cuda.synchronize()
    # the tile table: one entry per non-empty expert here (fewer than 128 rows each)
    live = [e for e in range(E) if goff[e + 1] > goff[e]]
    assert int(ntl) == len(live)
    assert tab[:len(live)].cpu().tolist() == [[e, int(goff[e]), int(goff[e + 1]), 0] for e in live]
    assert idx[0].tolist() == [1, 2, 4]
    val, ref = torch.topk(z[1:], top, -1)
    assert torch.equal(idx[1:].cpu().long(), ref)
    assert torch.allclose(wts[1:].cpu(), torch.softmax(val, -1), atol=1e-6)
    # the grouping: every pair sits in its expert's segment, and perm_tok / pair_pos are inverse views
    goff, perm, ppos, idx = goff.cpu(), perm.cpu(), ppos.cpu(), idx.cpu().reshape(-1)
    assert goff[0] == 0 and goff[-1] == T_ * top
    for p in range(T_ * top):
        e = int(idx[p])
        assert goff[e] <= ppos[p] < goff[e + 1] and perm[ppos[p]] == p // top
    assert sorted(ppos.tolist()) == list(range(T_ * top))


# ---- the grouped tensor-core GEMM behind routed experts, per-head projections and fp32 logits ----------
def test_grouped_gemm_experts_heads_and_f32(cuda):
    L, lib = _ops()
    g = torch.Generator().manual_seed(5)
    bf = torch.bfloat16
    # experts: rows sorted by group, uneven groups (one empty, one larger than a tile)
    E, N, K = 5, 192, 128
    counts = [37, 0, 300, 1, 130]
    P = sum(counts)
    A = torch.randn(P, K, generator=g).to(bf).to(cuda)
    W = (torch.randn(E * N, K, generator=g) * 0.1).to(bf).to(cuda)
    off = np.concatenate([[0], np.cumsum(counts)])
    tab = [[e, r, int(off[e + 1]), 0] for e in range(E) for r in range(int(off[e]), int(off[e + 1]), 128)]
    tabd = torch.tensor(tab, dtype=torch.int32, device=cuda)
    ntl = torch.tensor([len(tab)], dtype=torch.int32, device=cuda)
    C = torch.full((P, N), 9.0, dtype=bf, device=cuda)
    assert lib.b200q_gemm_grouped_ok(A.data_ptr(), K, 0, W.data_ptr(), C.data_ptr(), N, 0, N, K, 0)
    L.check(lib.b200q_gemm_grouped_bf16(A.data_ptr(), P, K, 0, W.data_ptr(), E, C.data_ptr(), N, 0, 0, N, K,
                                        tabd.data_ptr(), ntl.data_ptr(), P // 128 + E, 0, None))
    torch.cuda.synchronize()
    want = torch.cat([A[off[e]:off[e + 1]].float() @ W[e * N:(e + 1) * N].float().T for e in range(E)])
    assert rel_err(C.float().cpu().numpy(), want.cpu().numpy()) < 6e-3
    # heads: every head a column slice of A and of C, fp32 out into a wider row
    H, M, Kh, Nh, ldc, cgx = 3, 150, 64, 128, 3 * 136, 136
    A2 = torch.randn(M, H * (Kh + 8), generator=g).to(bf).to(cuda)
    W2 = (torch.randn(H * Nh, Kh, generator=g) * 0.1).to(bf).to(cuda)
    C2 = torch.full((M, ldc), 7.0, device=cuda)
    L.check(lib.b200q_linear_batched(A2.data_ptr(), H * (Kh + 8), Kh + 8, W2.data_ptr(), Nh * Kh, C2.data_ptr(), ldc,
                                     cgx, M, Nh, Kh, H, L.DTYPE_BF16, 1, None))
    torch.cuda.synchronize()
    for h in range(H):
        w = A2[:, h * (Kh + 8):h * (Kh + 8) + Kh].float() @ W2[h * Nh:(h + 1) * Nh].float().T
        assert rel_err(C2[:, h * cgx:h * cgx + Nh].cpu().numpy(), w.cpu().numpy()) < 1e-5
        assert float(C2[:, h * cgx + Nh:(h + 1) * cgx].min()) == 7.0        # the gap between slices is untouched


def test_tensor_core_shapes_through_the_model(cuda):
    """sizes that put every projection of the model on the tensor-core paths (multiples of 64), bf16"""
    spec = small_spec(width=128, vocab=192, layers=[
        attn(heads=2, dim=64, rot_dim=64, vdim=64, q_rank=64, kv_rank=128, window=40,
             ff="moe", ff_dim=64, n_experts=4, top_k=2, expert_limit=2.0, shared_dim=64, shared_limit=1.0),
        delta(heads=2, dim=64, rank=64, ff="dense", ff_dim=256),
        attn(heads=2, dim=64, rot_dim=64, vdim=64, q_rank=64, kv_rank=128, window=9, kv_from=0, **DENSE)])
    sd = checkpoint(spec, seed=31)
    toks = tokens(200, spec.vocab, 6)
    want = oracle_logits(spec, sd, toks)
    model, eng = build(spec, sd, torch.bfloat16)
    whole = eng.step_replay([(1, toks, list(range(len(toks))))])
    cut = replay_cut(eng, 2, toks, [130, 3, 40])
    rows = np.sqrt(((whole - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
    assert np.quantile(rows, 0.9) < BF16_TOL, float(np.quantile(rows, 0.9))
    rows = np.sqrt(((cut - whole) ** 2).mean(-1)) / np.sqrt((whole ** 2).mean(-1))
    assert np.quantile(rows, 0.9) < BF16_TOL
    eng.close()
    model.close()


# ---- latent attention kernel with made-up inputs: one key stands out ------------------------------------
def _latent_attn(cuda, qa, rows, pos, table, window, scale, R, P, bs=16, dtype=torch.float32):
    """qa [n, H, R+P] at positions pos of ONE sequence whose cached rows [L, R+P] lie in shuffled pages"""
    L, lib = _ops()
    n, H = qa.shape[0], qa.shape[1]
    n_blocks = int(max(table)) + 1
    cache = torch.full((n_blocks * bs, R + P), 1e4, dtype=dtype)  # whatever is not written is poison
    for j in range(rows.shape[0]):
        cache[table[j // bs] * bs + j % bs] = rows[j]
    bt = torch.tensor([table], dtype=torch.int32, device=cuda)
    out = torch.zeros(n, H, R, device=cuda, dtype=dtype)
    qd, cd = qa.to(cuda).contiguous(), cache.to(cuda)
    rs, ps = torch.zeros(n, dtype=torch.int32, device=cuda), torch.tensor(pos, dtype=torch.int32, device=cuda)
    L.check(lib.b200q_latent_attn(qd.data_ptr(), cd.data_ptr(), bt.data_ptr(), bt.shape[1], rs.data_ptr(),
                                  ps.data_ptr(), n, H, R, P, bs, window, scale, out.data_ptr(),
                                  L.DTYPE_F32 if dtype == torch.float32 else L.DTYPE_BF16, None))
    torch.cuda.synchronize()
    return out.float().cpu()


@pytest.mark.parametrize("window,H,R,P", [(0, 9, 64, 16), (70, 18, 128, 32), (64, 16, 192, 16), (5, 3, 64, 0),
                                          # (kv_rank + rot_dim) % 64 == 0: the variant with the query in registers
                                          (70, 16, 64, 64), (0, 9, 128, 64), (33, 20, 256, 64), (0, 5, 512, 64)])
def test_latent_attn_tensor_core_kernel(cuda, window, H, R, P):
    """the bf16 tensor-core kernel: random queries over hundreds of keys, and queries that single out one key
    (first key, chunk and page borders, window edge) — against the plain fp64 form on the same bf16 rows"""
    Lq, bs = 300, 16
    g = torch.Generator().manual_seed(6)
    rows = torch.randn(Lq, R + P, generator=g).to(torch.bfloat16)
    table = torch.randperm(Lq // bs + 1, generator=g).tolist()
    pos = [0, 1, 15, 16, 63, 64, 65, 127, 128, 129, 200, 299]
    qa = torch.randn(len(pos), H, R + P, generator=g) * 0.5
    got = _latent_attn(cuda, qa, rows, pos, table, window, 0.3, R, P, bs, torch.bfloat16)
    want = O.windowed_attention(qa.double(), rows.double(), rows[:, :R].double(), torch.tensor(pos), window, 0.3)
    assert rel_err(got.reshape(len(pos), -1), want.reshape(len(pos), -1)) < 2e-2
    unit = rows.float() / rows.float().norm(dim=-1, keepdim=True) ** 2
    for back in sorted({0, 1, 63, 64, 65, 128, max(window - 1, 0), window, window + 1}):
        ps = [p for p in pos if p - back >= 0]
        if not ps:
            continue
        q1 = torch.stack([unit[p - back] for p in ps])[:, None, :].repeat(1, H, 1) * 80.0
        got = _latent_attn(cuda, q1, rows, ps, table, window, 1.0, R, P, bs, torch.bfloat16)
        want = O.windowed_attention(q1.double(), rows.double(), rows[:, :R].double(), torch.tensor(ps), window, 1.0)
        assert rel_err(got.reshape(len(ps), -1), want.reshape(len(ps), -1)) < 2e-2, (window, back)


@pytest.mark.parametrize("window", [0, 1, 16, 17, 50])
def test_latent_attn_standout_key(cuda, window):
    """the query of every asked position points at ONE key: just inside the window, just outside it, on
    either side of a page border, the very first key, far back.  Inside: the output is that key's latent;
    outside: the key must not be seen at all."""
    R, P, H, Lq, bs = 20, 6, 9, 150, 16
    g = torch.Generator().manual_seed(3)
    rows = torch.randn(Lq, R + P, generator=g)
    rows = rows / rows.norm(dim=-1, keepdim=True)
    table = torch.randperm(Lq // bs + 1, generator=g).tolist()
    asked = [0, 1, 15, 16, 17, 31, 32, 49, 50, 51, 100, 149]
    for back in sorted({0, 1, 15, 16, 17, 49, 50, 51, 99, max(window - 1, 0), window, window + 1}):
        pos = [p for p in asked if p - back >= 0]
        if not pos:
            continue
        qa = torch.stack([rows[p - back] for p in pos])[:, None, :].repeat(1, H, 1) * 60.0   # score 60 vs |.| <~ 20
        qa = qa * torch.linspace(0.9, 1.1, H)[None, :, None]
        got = _latent_attn(cuda, qa, rows, pos, table, window, 1.0, R, P, bs)
        want = O.windowed_attention(qa.double(), rows.double(), rows[:, :R].double(), torch.tensor(pos), window, 1.0)
        assert rel_err(got.reshape(len(pos), -1), want.reshape(len(pos), -1)) < 1e-4, (window, back)
        seen = window == 0 or back < window
        hit = (got - rows[[p - back for p in pos], :R][:, None, :]).abs().max()
        assert (hit < 1e-3) == seen, (window, back, float(hit))


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("D", [24, 32, 64, 128])
def test_delta_rule_op_state_slots(cuda, D, split):
    """the recurrence kernel alone: two sequences in one launch, one continuing from its slot and one starting
    (position 0) in a slot that holds another sequence's leftovers"""
    L, lib = _ops()
    H, Rk, eps = 3, 4 if D < 64 else 37, 1e-5
    HD, NP = H * D, 5 * H * D + Rk
    g = torch.Generator().manual_seed(4)
    n_a, n_b, n_a2 = 13, 7, 5
    proj = torch.randn(n_a + n_b + n_a2, NP, generator=g)
    w2, w0, ab, on = (torch.randn(HD, Rk, generator=g), torch.randn(HD, generator=g), torch.randn(HD, generator=g) * 0.3,
                      1 + 0.1 * torch.randn(HD, generator=g))

    def reference(rows):
        p = proj[rows].double()
        r, k, v, gt, a = [p[:, i * HD:(i + 1) * HD] for i in range(5)]
        z = torch.tanh(p[:, 5 * HD:]) @ w2.double().T + w0.double()
        w = torch.exp(-np.exp(-0.5) * torch.sigmoid(z))
        a = torch.sigmoid(a + ab.double())
        out = torch.zeros(len(rows), HD, dtype=torch.float64)
        for h in range(H):
            s = slice(h * D, (h + 1) * D)
            o, _ = O.delta_rule_steps(r[:, s], k[:, s], v[:, s], w[:, s], a[:, s])
            out[:, s] = O.rms_unit(o, eps)
        return out * on.double() * torch.sigmoid(gt)

    slot_floats = H * D * D + 10                                  # a slot may be wider than this layer's part
    state = torch.full((3, slot_floats), 7.0, device=cuda)        # leftovers everywhere
    out = torch.zeros(proj.shape[0], HD, device=cuda)
    scratch = torch.zeros(6 * proj.shape[0] * HD, device=cuda)    # the three-launch form's per-token vectors
    dev = lambda t: t.to(cuda).contiguous()
    pj, w2d, w0d, abd, ond = dev(proj), dev(w2), dev(w0), dev(ab), dev(on)

    def run(desc):
        sd_ = torch.tensor(desc, dtype=torch.int32, device=cuda)
        L.check(lib.b200q_delta_rule(pj.data_ptr(), NP, w2d.data_ptr(), w0d.data_ptr(), abd.data_ptr(), ond.data_ptr(),
                                     state.data_ptr(), slot_floats, sd_.data_ptr(), len(desc), H, D, Rk, eps,
                                     out.data_ptr(), L.DTYPE_F32, scratch.data_ptr() if split else None,
                                     proj.shape[0], None))
        torch.cuda.synchronize()

    run([[0, n_a, 0, 2], [n_a, n_b, 0, 0]])                       # a in slot 2, b in slot 0, both from position 0
    run([[n_a + n_b, n_a2, n_a, 2]])                              # a goes on from its slot
    rows_a = list(range(n_a)) + list(range(n_a + n_b, n_a + n_b + n_a2))
    assert rel_err(out.cpu()[rows_a].numpy(), reference(rows_a).numpy()) < 1e-4
    assert rel_err(out.cpu()[n_a:n_a + n_b].numpy(), reference(list(range(n_a, n_a + n_b))).numpy()) < 1e-4
    assert float(state[1].min()) == 7.0 and float(state[0, H * D * D:].min()) == 7.0   # nothing else was touched


# ---- the whole model through the engine ----------------------------------------------------------------
@pytest.fixture(scope="module")
def small(cuda):
    spec = small_spec()
    sd = checkpoint(spec, seed=21)
    return spec, sd


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_every_layer(cuda, small, dtype):
    spec, sd = small
    toks = tokens(70, spec.vocab, 1)
    model, eng = build(spec, sd, dtype)
    tap = torch.zeros(spec.n_layers, len(toks), spec.width, device=cuda)
    model.set_layer_tap(tap)
    got = eng.step_replay([(1, toks, list(range(len(toks))))])
    model.set_layer_tap(None)
    want, stream = O.forward(spec.to_config(), sd, toks, torch.float64, keep_layers=True)
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    for i in range(spec.n_layers):
        assert rel_err(tap[i].cpu().numpy(), stream[i].numpy()) < tol, f"layer {i}"
    assert rel_err(got, want.numpy()) < tol
    eng.close()
    model.close()


@pytest.mark.parametrize("cuts", [[], [1, 1], [2, 2, 2, 3, 5], [16, 16, 1, 15], [17, 2, 31], [64], [7, 90]])
def test_portions_and_token_by_token(cuda, small, cuts):
    """a prompt cut into portions (down to two tokens, across page and window edges) and then decoded token by
    token gives the logits of the whole prompt; [] = every token alone from the first"""
    spec, sd = small
    toks = tokens(100, spec.vocab, 2)
    want = oracle_logits(spec, sd, toks)
    model, eng = build(spec, sd)
    got = replay_cut(eng, 1, toks, cuts)
    assert rel_err(got, want) < F32_TOL
    eng.close()
    model.close()


def test_long_decoding_past_windows_and_pages(cuda, small):
    spec, sd = small
    toks = tokens(330, spec.vocab, 3)
    want = oracle_logits(spec, sd, toks)
    for dtype, tol in ((torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)):
        model, eng = build(spec, sd, dtype)
        got = replay_cut(eng, 1, toks, [3])
        assert rel_err(got, want) < tol
        eng.close()
        model.close()


def test_mixed_batches_pages_and_slots_reused(cuda, small):
    """up to three live requests in a pool too small for all of them: portions of some beside single tokens of
    others, requests that sit a step out, finished requests whose pages and state slot go to the next one.
    Every request must come out as if it had run alone."""
    spec, sd = small
    rng = np.random.default_rng(7)
    lens = [37, 5, 64, 18, 1, 49, 33, 2, 80]
    reqs = {i: tokens(n, spec.vocab, 100 + i) for i, n in enumerate(lens)}
    want = {i: oracle_logits(spec, sd, t) for i, t in reqs.items()}
    model, eng = build(spec, sd, max_tokens=160, max_seqs=3, num_blocks=13)   # 208 token places for 289 tokens
    state0 = model.state.clone()
    model.state.fill_(3.0)                                                     # slots start dirty
    model.kv.view(torch.float32).fill_(1e3)
    got = {i: [] for i in reqs}
    at = {i: 0 for i in reqs}
    waiting, live = list(reqs), []
    while waiting or live:
        while waiting and len(live) < 3:
            need = sum((len(reqs[i]) + 15) // 16 for i in live) + (len(reqs[waiting[0]]) + 15) // 16
            if need > 13:
                break
            live.append(waiting.pop(0))
        entries, done = [], []
        for i in live:
            if len(live) > 1 and rng.random() < 0.2:
                continue                                                       # sits this step out
            left = len(reqs[i]) - at[i]
            n = min(left, int(rng.choice([1, 1, 2, 3, 9, 16, 40])))
            entries.append((i, reqs[i][at[i]:at[i] + n], list(range(n))))
        if not entries:
            continue
        out = eng.step_replay(entries)
        row = 0
        for i, t, w in entries:
            got[i].append(out[row:row + len(w)])
            row += len(w)
            at[i] += len(t)
            if at[i] == len(reqs[i]):
                done.append(i)
        for i in done:
            eng.abort(i)
            live.remove(i)
    for i in reqs:
        assert rel_err(np.concatenate(got[i]), want[i]) < F32_TOL, f"request {i}"
    assert eng.stats().free_blocks == 13
    eng.close()
    model.close()


def test_pool_too_small_is_refused_and_leaves_the_request_intact(cuda, small):
    from llmq_b200.lib import B200QError
    spec, sd = small
    model, eng = build(spec, sd, max_tokens=64, max_seqs=2, num_blocks=2)
    toks = tokens(40, spec.vocab, 9)
    a = eng.step_replay([(1, toks[:20], [19])])
    with pytest.raises(B200QError):
        eng.step_replay([(1, toks[20:], [0]), (2, toks[:17], [0])])           # would need 3 + 2 pages
    b = eng.step_replay([(1, toks[20:32], list(range(12)))])                  # request 1 goes on where it was
    want = oracle_logits(spec, sd, toks[:32])
    assert rel_err(np.concatenate([a, b]), want[19:]) < F32_TOL
    eng.close()
    model.close()


# ---- generation through the engine's own scheduler, sampler and model directory reader ----------------
def _generate(eng, prompts, n_new):
    for i, p in enumerate(prompts):
        eng.add_request(i, p, n_new, ignore_eos=True)
    outs = {i: [] for i in range(len(prompts))}
    while eng.has_work():
        ids, toks, _ = eng.step()
        for i, t in zip(ids.tolist(), toks.tolist()):
            outs[i].append(t)
    return outs


def test_greedy_generation_from_a_model_directory(cuda, small, tmp_path):
    """config.json + model.safetensors on disk -> resolve_model -> NativeModel -> Engine.add_request/step:
    chunked prefill under a small token budget, continuous batching of unequal requests, decode-only steps
    (replayed from CUDA graphs), more requests than state slots"""
    from llmq_b200.model import Engine, NativeModel, checkpoint_engine_weights, resolve_model
    from llmq_b200.ramopel import save_checkpoint

    spec, sd = small
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(spec.to_config()))
    save_checkpoint(str(d / "model.safetensors"), sd)
    spec2, model_dir = resolve_model(str(d))
    assert spec2.layers == spec.layers and spec2.layered
    prompts = [tokens(n, spec.vocab, 40 + n) for n in (3, 41, 1, 26, 17, 9)]
    n_new = 24
    model = NativeModel(spec2, checkpoint_engine_weights(spec2, model_dir), max_tokens=32, max_seqs=4,
                        max_model_len=128, num_blocks=24, dtype=torch.float32)
    eng = Engine(model, max_num_seqs=4, max_num_batched_tokens=32)
    outs = _generate(eng, prompts, n_new)
    cfg = spec.to_config()
    for i, p in enumerate(prompts):
        assert outs[i] == O.greedy(cfg, sd, p, n_new), f"request {i}"
    eng.close()
    model.close()


def test_greedy_generation_bf16_matches_its_own_replay(cuda, small):
    """bf16 serving: what the scheduler generates is what a replay of the same tokens predicts (sampling,
    async stepping and graphs change nothing), and the logits stay within rounding of the oracle"""
    spec, sd = small
    prompts = [tokens(n, spec.vocab, 60 + n) for n in (12, 30)]
    model, eng = build(spec, sd, torch.bfloat16, max_tokens=64)
    outs = _generate(eng, prompts, 20)
    fresh_model, fresh = build(spec, sd, torch.bfloat16, max_tokens=64)
    for i, p in enumerate(prompts):
        full = p + outs[i]
        lg = eng.step_replay([(100 + i, full, list(range(len(full))))])
        eng.abort(100 + i)
        # the engine that has generated (used pages and slots, graphs) computes what a new one does
        again = fresh.step_replay([(1, full, list(range(len(full))))])
        fresh.abort(1)
        assert rel_err(lg, again) < 1e-6
        # against the oracle a bf16 router may settle a near-tie the other way on a few rows: most rows close
        want = oracle_logits(spec, sd, full)
        rows = np.sqrt(((lg - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
        assert np.quantile(rows, 0.75) < BF16_TOL
        top2 = np.sort(lg[len(p) - 1:-1], -1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05 * np.abs(lg).max()         # skip near-ties of bf16 rounding
        pred = lg[len(p) - 1:-1].argmax(-1)
        assert (pred[clear] == np.asarray(outs[i])[clear]).all()
    fresh.close()
    fresh_model.close()
    eng.close()
    model.close()
