"""GPU tests of the Noridra path: the engine (scheduler, paged key cache, state slots, kernels) against
oracle/noridra.py — a plain fp64 restatement that recomputes every position from the tokens, with no cache,
no state and no batching.  The configurations are small, differ from one another in every size, and are
drawn here; the fp32 engine is held to a tight bound, the bf16 engine to a rounding-sized one."""
import json

import numpy as np
import pytest
import torch

from oracle import noridra as O
from tests.noridra_util import MOE, MOE_ALL, MOE_ONE, attn, checkpoint, delta, rel_err, scan, small_spec, tokens

pytestmark = pytest.mark.gpu
F32_TOL, BF16_TOL = 2e-4, 8e-2


def build(spec, sd, dtype=torch.float32, max_tokens=512, max_seqs=4, num_blocks=None):
    from llmq_b200.model import BLOCK_SIZE, Engine, NativeModel

    nb = num_blocks or (max_tokens // BLOCK_SIZE + max_seqs)
    model = NativeModel(spec, spec.engine_weights(sd), max_tokens=max_tokens, max_seqs=max_seqs,
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


def check_close(got, want, dtype, what=""):
    """fp32: every row within the tight bound.  bf16: a router may settle a near-tie the other way on a few
    rows (another expert answers there), so nine rows in ten within the rounding-sized bound"""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    rows = np.sqrt(((got - want) ** 2).mean(-1)) / (np.sqrt((want ** 2).mean(-1)) + 1e-30)
    if dtype == torch.float32:
        assert rows.max() < F32_TOL, what
    else:
        assert np.quantile(rows, 0.9) < BF16_TOL, what


def _ops():
    from llmq_b200 import lib as L
    return L, L.load()


# ---- every mechanism alone: a one-layer model around it --------------------------------------------------
ONE_LAYER = {
    "gated_delta": [delta()],
    "gated_delta_equal_heads_wide": [delta(heads=3, kv_heads=3, dim=72, vdim=40, conv=4)],
    "gated_delta_one_tap": [delta(heads=2, kv_heads=1, dim=8, vdim=33, conv=1)],
    "chunk_attention": [attn()],
    "chunk_attention_no_state_at_all": [attn(heads=4, kv_heads=4, dim=16, chunk=11)],   # one-tap input convolutions
    "chunk_attention_many_heads_per_key": [attn(heads=18, kv_heads=2, dim=8, chunk=7)],
    "chunk_attention_plain_causal": [attn(heads=2, kv_heads=1, dim=72, softcap=0.0, chunk=0)],
    "selective_scan": [scan()],
    "selective_scan_wide_state": [scan(inner=200, state=40, dt_rank=9, conv=3)],
    "experts_two": [scan(inner=32, state=4, dt_rank=2, conv=2, **MOE)],
    "experts_one": [scan(inner=32, state=4, dt_rank=2, conv=2, **MOE_ONE)],
    "experts_all_chosen": [scan(inner=32, state=4, dt_rank=2, conv=2, **MOE_ALL)],
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mechanism_alone(cuda, name, dtype):
    spec = small_spec(width=80, vocab=97, layers=ONE_LAYER[name], groups=5 if "experts" in name else 1,
                      taps=1 if name in ("gated_delta", "chunk_attention_no_state_at_all") else 4)
    sd = checkpoint(spec, seed=11)
    toks = tokens(45, spec.vocab, 5)
    model, eng = build(spec, sd, dtype)
    tap = torch.zeros(spec.n_layers, len(toks), spec.width, device=cuda)
    model.set_layer_tap(tap)
    got = eng.step_replay([(1, toks, list(range(len(toks))))])
    model.set_layer_tap(None)
    stream = []
    want = O.forward(spec.to_config(), sd, toks, torch.float64, stream)
    check_close(tap.cpu().numpy()[-1], stream[-1].numpy(), dtype, name)
    check_close(got, want.numpy(), dtype, name)
    eng.close()
    model.close()


# ---- op level: made-up inputs that make a fault show ----------------------------------------------------
def _attention_op(cuda, qs, keys, chunk, cap, scale, r1, r2, dtype, block_size=16, shuffle_seed=0):
    """run b200q_chunk_attn for one sequence of T tokens whose raw keys lie in a paged cache with shuffled
    pages; the gate is wide open (logit 30)"""
    L, lib = _ops()
    T, H, D = qs.shape
    G = keys.shape[1]
    tdt = torch.float32 if dtype == L.DTYPE_F32 else torch.bfloat16
    nb = (T + block_size - 1) // block_size
    rng = np.random.default_rng(shuffle_seed)
    pages = rng.permutation(nb + 3)[:nb].astype(np.int32)
    cache = torch.full(((nb + 3) * block_size, G * D), 1e4, dtype=tdt, device=cuda)   # unused places hold garbage
    for t in range(T):
        cache[int(pages[t // block_size]) * block_size + t % block_size] = keys[t].reshape(-1).to(tdt)
    bt = torch.tensor(pages, device=cuda).reshape(1, -1).contiguous()
    row_seq = torch.zeros(T, dtype=torch.int32, device=cuda)
    pos = torch.arange(T, dtype=torch.int32, device=cuda)
    gate = torch.full((T, H * D), 30.0, dtype=tdt, device=cuda)
    out = torch.zeros(T, H * D, dtype=tdt, device=cuda)
    qd = qs.to(cuda).float().contiguous()
    r1d, r2d = r1.to(cuda).float(), r2.to(cuda).float()
    L.check(lib.b200q_chunk_attn(qd.data_ptr(), cache.data_ptr(), bt.data_ptr(), nb, row_seq.data_ptr(), pos.data_ptr(),
                                 T, H, G, D, block_size, chunk, scale, cap, r1d.data_ptr(), r2d.data_ptr(),
                                 gate.data_ptr(), H * D, 1e-6, out.data_ptr(), dtype, None))
    torch.cuda.synchronize()
    return out.float().cpu().reshape(T, H, D)


def _standout(T, H, G, D, marks, seed):
    """small random queries and keys; at every marked position the key points along the (shared) query
    direction of its group and is large, so whoever sees it is dominated by it"""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(G, D, generator=g)
    u = u / u.norm(dim=-1, keepdim=True)
    qs = 0.05 * torch.randn(T, H, D, generator=g) + 6.0 * u.repeat_interleave(H // G, 0)[None]
    keys = 0.3 * torch.randn(T, G, D, generator=g)
    keys = keys - (keys * u[None]).sum(-1, keepdim=True) * u[None] * 1.5         # the crowd points away a little
    for i, m in enumerate(marks):   # every marked key has its own length, so each one gives another output
        keys[m] = (8.0 + 5.0 * (i % 7)) * u + 0.1 * torch.randn(G, D, generator=g)
    return qs.bfloat16().float(), keys.bfloat16().float()


@pytest.mark.parametrize("dtype_name", ["f32", "bf16"])
@pytest.mark.parametrize("chunk", [50, 33, 16, 0])
def test_attention_edges_of_chunks_pages_and_tiles(cuda, dtype_name, chunk):
    """standout keys sit just inside and just outside every chunk edge, at page borders (16) and at the
    borders of the kernel's key tiles (32 from the chunk's first key), and far back among hundreds"""
    L, _ = _ops()
    T, H, G, D = 310, 6, 2, 24
    marks = {3, 15, 16, 17, 31, 32, 33, 47, 48, 63, 64, 65, 255, 256, 257}
    if chunk:
        for e in range(chunk, T, chunk):
            marks |= {e - 1, e, e + 31, e + 32}
    marks = sorted(m for m in marks if m < T)
    qs, keys = _standout(T, H, G, D, marks, 3)
    r1, r2 = torch.linspace(0.2, 0.9, H), torch.linspace(0.1, 1.5, H)
    kn = keys / torch.sqrt((keys * keys).mean(-1, keepdim=True) + 1e-6)
    want = O.sink_attention(qs.double(), kn.double(), keys.double(), r1.double(), r2.double(), 0.2, 9.0, chunk)
    got = _attention_op(cuda, qs, keys, chunk, 9.0, 0.2, r1, r2, L.DTYPE_F32 if dtype_name == "f32" else L.DTYPE_BF16)
    tol = 2e-5 if dtype_name == "f32" else 2e-2
    assert rel_err(got.reshape(T, -1).numpy(), want.reshape(T, -1).numpy()) < tol
    # the made-up keys do what they are for: with every chunk edge moved by one token (a dummy token in
    # front shifts the count) the rows behind an edge come out clearly different
    if chunk:
        sh = lambda x: torch.cat([x[:1], x]).double()
        off = O.sink_attention(sh(qs), sh(kn), sh(keys), r1.double(), r2.double(), 0.2, 9.0, chunk)[1:]
        rows = [e + d for e in range(chunk, T - 2, chunk) for d in (0, 1)]
        diff = (off[rows] - want[rows]).reshape(len(rows), -1).norm(dim=-1) / want[rows].reshape(len(rows), -1).norm(dim=-1)
        assert float(diff.median()) > 0.05


@pytest.mark.parametrize("D,H,G", [(64, 4, 1), (128, 8, 2), (64, 18, 2), (128, 3, 3)])
@pytest.mark.parametrize("chunk", [50, 0])
def test_attention_tensor_core_form_in_portions(cuda, D, H, G, chunk):
    """the tile kernel (bf16 cache, head size 64 / 128), fed one sequence in portions of 1 to 150 tokens whose
    16-token tiles straddle chunk edges, against the oracle; two sequences share a step at the end"""
    L, lib = _ops()
    T, bs = 310, 16
    marks = sorted({3, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256} | ({e + d for e in range(chunk, T, chunk) for d in (-1, 0)} if chunk else set()))
    qs, keys = _standout(T, H, G, D, [m for m in marks if m < T], 9)
    r1, r2 = torch.linspace(0.2, 0.9, H), torch.linspace(0.1, 1.5, H)
    kn = keys / torch.sqrt((keys * keys).mean(-1, keepdim=True) + 1e-6)
    want = O.sink_attention(qs.double(), kn.double(), keys.double(), r1.double(), r2.double(), 0.2, 9.0, chunk)
    nb = (T + bs - 1) // bs
    pages = np.random.default_rng(1).permutation(2 * nb + 3)[:2 * nb].astype(np.int32).reshape(2, nb)
    cache = torch.full(((2 * nb + 3) * bs, G * D), 1e4, dtype=torch.bfloat16, device=cuda)
    for t in range(T):      # both sequences hold the same keys, in different pages
        for q in range(2):
            cache[int(pages[q, t // bs]) * bs + t % bs] = keys[t].reshape(-1).bfloat16()
    bt = torch.tensor(pages, device=cuda).contiguous()
    r1d, r2d = r1.to(cuda), r2.to(cuda)
    got = torch.zeros(2, T, H * D)

    def run(parts):   # parts: [(sequence, first position, tokens)]
        rows = sum(n for _, _, n in parts)
        q = torch.cat([qs[p0:p0 + n] for _, p0, n in parts]).to(cuda).float().contiguous()
        desc, rseq, pos, at = [], [], [], 0
        for k, (sq, p0, n) in enumerate(parts):
            desc.append([at, n, p0, k])
            rseq += [k] * n
            pos += list(range(p0, p0 + n))
            at += n
        btab = torch.stack([bt[sq] for sq, _, _ in parts]).contiguous()
        dd = torch.tensor(desc, dtype=torch.int32, device=cuda)
        rs, ps = torch.tensor(rseq, dtype=torch.int32, device=cuda), torch.tensor(pos, dtype=torch.int32, device=cuda)
        gate = torch.full((rows, H * D), 30.0, dtype=torch.bfloat16, device=cuda)
        out = torch.zeros(rows, H * D, dtype=torch.bfloat16, device=cuda)
        L.check(lib.b200q_chunk_attn_seq(q.data_ptr(), cache.data_ptr(), btab.data_ptr(), nb, rs.data_ptr(), ps.data_ptr(),
                                         dd.data_ptr(), len(parts), rows, H, G, D, bs, chunk, 0.2, 9.0, r1d.data_ptr(),
                                         r2d.data_ptr(), gate.data_ptr(), H * D, 1e-6, out.data_ptr(), L.DTYPE_BF16, None))
        torch.cuda.synchronize()
        at = 0
        for sq, p0, n in parts:
            got[sq, p0:p0 + n] = out[at:at + n].float().cpu()
            at += n

    at = 0
    for n in [1, 1, 2, 45, 17, 1, 150, 33]:          # sequence 0 alone: 250 tokens
        run([(0, at, n)])
        at += n
    run([(1, 0, 201), (0, 250, 1)])                 # a long portion of sequence 1 beside one token of sequence 0
    run([(0, 251, 59), (1, 201, 109)])
    for sq in range(2):
        assert rel_err(got[sq].numpy(), want.reshape(T, -1).numpy()) < 2e-2, sq


def test_attention_sink_takes_the_weight_when_no_key_fits(cuda):
    """all keys point away from the query: the scores sit at minus the cap, the silent zero-score term holds
    nearly all of the weight and the output is nearly zero (without that term it would be a mean of keys)"""
    L, _ = _ops()
    T, H, G, D = 70, 4, 2, 16
    g = torch.Generator().manual_seed(4)
    u = torch.randn(G, D, generator=g)
    u = u / u.norm(dim=-1, keepdim=True)
    qs = (8.0 * u.repeat_interleave(H // G, 0))[None].repeat(T, 1, 1)
    keys = -5.0 * u[None] + 0.05 * torch.randn(T, G, D, generator=g)
    r1, r2 = torch.zeros(H), torch.zeros(H)
    got = _attention_op(cuda, qs, keys, 0, 20.0, 1.0, r1, r2, L.DTYPE_F32)
    kn = keys / torch.sqrt((keys * keys).mean(-1, keepdim=True) + 1e-6)
    want = O.sink_attention(qs.double(), kn.double(), keys.double(), r1.double(), r2.double(), 1.0, 20.0, 0)
    assert float(want.abs().max()) < 1e-5 and float(got.abs().max()) < 1e-5
    # and with keys that fit, the sink's share is what the oracle says
    got = _attention_op(cuda, qs * 0.02, -keys, 0, 20.0, 1.0, r1, r2, L.DTYPE_F32)
    want = O.sink_attention(qs.double() * 0.02, -kn.double(), -keys.double(), r1.double(), r2.double(), 1.0, 20.0, 0)
    assert rel_err(got.reshape(T, -1).numpy(), want.reshape(T, -1).numpy()) < 2e-5


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_convolution_carries_its_inputs_across_portions(cuda, taps):
    """two sequences in slots 2 and 0, fed in portions of 1, 2, taps-1 and more tokens in interleaved steps,
    slots dirty at the start: every output equals the convolution over the whole sequence"""
    L, lib = _ops()
    C_, nslots = 37, 3
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C_, taps, generator=g)
    bias = torch.randn(C_, generator=g)
    seqs = {2: torch.randn(29, C_, generator=g), 0: torch.randn(17, C_, generator=g)}
    stride = (taps - 1) * C_ + 5
    state = torch.full((nslots * stride + 8,), 9.0, device=cuda)
    wd, bd = w.to(cuda).contiguous(), bias.to(cuda)
    got = {s: [] for s in seqs}
    at = {s: 0 for s in seqs}
    plan = [{2: 1, 0: 2}, {2: 2}, {2: max(taps - 1, 1), 0: 1}, {0: 1}, {2: 9, 0: 6}, {2: 1, 0: 1}, {2: 50, 0: 50}]
    for step in plan:
        rows, desc, rseq = [], [], []
        for si, (slot, n) in enumerate(step.items()):
            n = min(n, seqs[slot].shape[0] - at[slot])
            if n <= 0:
                continue
            desc.append([len(rows), n, at[slot], slot])
            rseq += [len(desc) - 1] * n
            rows += [seqs[slot][at[slot] + i] for i in range(n)]
        if not rows:
            continue
        x = torch.stack(rows).to(cuda).contiguous()
        y = torch.zeros_like(x)
        dd = torch.tensor(desc, dtype=torch.int32, device=cuda)
        rs = torch.tensor(rseq, dtype=torch.int32, device=cuda)
        L.check(lib.b200q_causal_conv(x.data_ptr(), C_, 1, wd.data_ptr(), bd.data_ptr(), C_, taps, 1, 0,
                                      state.data_ptr(), stride, dd.data_ptr(), rs.data_ptr(), len(desc), y.data_ptr(),
                                      C_, 1, x.shape[0], L.DTYPE_F32, None))
        torch.cuda.synchronize()
        for (r0, n, _, slot) in desc:
            got[slot].append(y[r0:r0 + n].cpu())
            at[slot] += n
    for slot, x in seqs.items():
        want = torch.nn.functional.silu(O.causal_conv(x.double(), w.double(), bias.double()))
        assert rel_err(torch.cat(got[slot]).numpy(), want.numpy()) < 1e-5, slot
    assert float(state[stride:2 * stride].min()) == 9.0            # slot 1 was nobody's


def test_router_sigmoid_scores_and_ties(cuda):
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
    L.check(lib.b200q_moe_route_ex(zc.data_ptr(), T_, E, top, 1, idx.data_ptr(), wts.data_ptr(), goff.data_ptr(),
                                   perm.data_ptr(), ppos.data_ptr(), None, None, None))
    torch.cuda.synchronize()
    assert idx[0].tolist() == [1, 2, 4]
    val, ref = torch.topk(z[1:], top, -1)
    assert torch.equal(idx[1:].cpu().long(), ref)
    assert torch.allclose(wts[1:].cpu(), torch.sigmoid(val), atol=1e-6)    # not renormalised
    # the scaled inputs land in expert order
    W = 24
    h = torch.randn(T_, W, generator=torch.Generator().manual_seed(3)).to(cuda)
    dst = torch.zeros(T_ * top, W, device=cuda)
    L.check(lib.b200q_scatter_scaled_rows(h.data_ptr(), ppos.data_ptr(), wts.data_ptr(), top, dst.data_ptr(), T_, W,
                                          L.DTYPE_F32, None))
    torch.cuda.synchronize()
    for p in range(T_ * top):
        e = int(idx.reshape(-1)[p])
        assert goff[e] <= ppos[p] < goff[e + 1]
        assert torch.allclose(dst[int(ppos[p])], h[p // top] * wts.reshape(-1)[p])


@pytest.mark.parametrize("groups", [1, 3, 8])
def test_group_norm_op(cuda, groups):
    L, lib = _ops()
    n, W = 11, 96
    g = torch.Generator().manual_seed(groups)
    x, add, ls, w = torch.randn(n, W, generator=g), torch.randn(n, W, generator=g), torch.randn(W, generator=g), torch.randn(W, generator=g)
    x[:, : W // groups] *= 30.0                                   # one part much larger: a norm over the whole row fails
    xd, ad, lsd, wd = x.to(cuda), add.to(cuda), ls.to(cuda), w.to(cuda)
    L.check(lib.b200q_group_rmsnorm(xd.data_ptr(), None, ad.data_ptr(), None, 0, lsd.data_ptr(), 1.7, wd.data_ptr(), groups,
                                    1e-5, xd.data_ptr(), None, n, W, L.DTYPE_F32, None))   # in place
    torch.cuda.synchronize()
    want = O.group_norm(1.7 * x.double() + ls.double() * add.double(), w.double(), groups, 1e-5)
    assert rel_err(xd.cpu().numpy(), want.numpy()) < 1e-5


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
    stream = []
    want = O.forward(spec.to_config(), sd, toks, torch.float64, stream)
    for i in range(spec.n_layers):
        check_close(tap[i].cpu().numpy(), stream[i].numpy(), dtype, f"layer {i}")
    check_close(got, want.numpy(), dtype)
    eng.close()
    model.close()


@pytest.mark.parametrize("cuts", [[], [1, 1], [2, 2, 2, 3, 5], [16, 16, 1, 15], [19, 2, 21], [20, 20, 2], [64], [7, 90]])
def test_portions_and_token_by_token(cuda, small, cuts):
    """a prompt cut into portions (down to two tokens, across page and chunk edges) and then decoded token by
    token gives the logits of the whole prompt; [] = every token alone from the first"""
    spec, sd = small
    toks = tokens(100, spec.vocab, 2)
    want = oracle_logits(spec, sd, toks)
    model, eng = build(spec, sd)
    got = replay_cut(eng, 1, toks, cuts)
    assert rel_err(got, want) < F32_TOL
    eng.close()
    model.close()


def test_long_decoding_past_chunks_and_pages(cuda, small):
    spec, sd = small
    toks = tokens(330, spec.vocab, 3)
    want = oracle_logits(spec, sd, toks)
    for dtype, tol in ((torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)):
        model, eng = build(spec, sd, dtype)
        got = replay_cut(eng, 1, toks, [3])
        check_close(got, want, dtype)
        eng.close()
        model.close()


def test_mixed_batches_pages_and_slots_reused(cuda, small):
    """up to three live requests in a pool too small for all of them: portions of some beside single tokens of
    others, requests that sit a step out, finished requests whose pages and state slot go to the next one
    (pool and slots start dirty).  Every request must come out as if it had run alone."""
    spec, sd = small
    rng = np.random.default_rng(7)
    lens = [37, 5, 64, 18, 1, 49, 33, 2, 80]
    reqs = {i: tokens(n, spec.vocab, 100 + i) for i, n in enumerate(lens)}
    want = {i: oracle_logits(spec, sd, t) for i, t in reqs.items()}
    model, eng = build(spec, sd, max_tokens=160, max_seqs=3, num_blocks=13)   # 208 token places for 289 tokens
    model.state.fill_(3.0)
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


def test_other_sizes_power_of_two_everything(cuda):
    """sizes the tensor-core paths take (multiples of 64) and several experts per token, in bf16 and fp32"""
    layers = [delta(heads=4, kv_heads=4, dim=64, vdim=64, conv=4, ff="moe", ff_dim=128, n_experts=8, top_k=2),
              attn(heads=4, kv_heads=1, dim=64, chunk=64, ff="moe", ff_dim=64, n_experts=4, top_k=4),
              scan(inner=256, state=16, dt_rank=8, conv=4, ff="moe", ff_dim=128, n_experts=8, top_k=1)]
    spec = small_spec(width=128, vocab=256, layers=layers, groups=4, taps=2, alpha=2.0)
    sd = checkpoint(spec, seed=5)
    toks = tokens(150, spec.vocab, 8)
    want = oracle_logits(spec, sd, toks)
    for dtype, tol in ((torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)):
        model, eng = build(spec, sd, dtype)
        got = replay_cut(eng, 1, toks, [130, 2, 9])
        check_close(got, want, dtype)
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
    from llmq_b200.noridra import save_checkpoint

    spec, sd = small
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(spec.to_config()))
    save_checkpoint(str(d / "model.safetensors"), sd)
    spec2, model_dir = resolve_model(str(d))
    assert spec2.layers == spec.layers and spec2.layered and spec2.arch == "noridra"
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
    async stepping and graphs change nothing)"""
    spec, sd = small
    prompts = [tokens(n, spec.vocab, 60 + n) for n in (12, 30)]
    model, eng = build(spec, sd, torch.bfloat16, max_tokens=64)
    outs = _generate(eng, prompts, 20)
    fresh_model, fresh = build(spec, sd, torch.bfloat16, max_tokens=64)
    for i, p in enumerate(prompts):
        full = p + outs[i]
        lg = eng.step_replay([(100 + i, full, list(range(len(full))))])
        eng.abort(100 + i)
        again = fresh.step_replay([(1, full, list(range(len(full))))])
        fresh.abort(1)
        assert rel_err(lg, again) < 1e-6
        top2 = np.sort(lg[len(p) - 1:-1], -1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05 * np.abs(lg).max()         # skip near-ties of bf16 rounding
        pred = lg[len(p) - 1:-1].argmax(-1)
        assert (pred[clear] == np.asarray(outs[i])[clear]).all()
    fresh.close()
    fresh_model.close()
    eng.close()
    model.close()
