"""CPU tests of the Ramopel host code: the config reader, the checkpoint file reader/writer, the mapping of
checkpoint tensors to engine weights, the oracle's own consistency, and replayed steps on the real C++
scheduler in dry-run mode (pages and state slots handed out, given back and used again)."""
import ctypes as C
import json

import numpy as np
import pytest
import torch

from llmq_b200 import lib as L
from llmq_b200 import ramopel as R
from oracle import ramopel as O
from tests.ramopel_util import attn, checkpoint, delta, small_spec, tokens, DENSE, MOE


def test_config_round_trip_and_sizes_from_tensors(tmp_path):
    spec = small_spec()
    sd = checkpoint(spec, 1)
    path = str(tmp_path / "model.safetensors")
    R.save_checkpoint(path, sd)
    cfg = json.loads(json.dumps(spec.to_config()))
    assert "decay_rank" not in json.dumps(cfg)                       # that size comes from a tensor's shape
    back = R.RamopelSpec.from_config(cfg, R.checkpoint_shapes(path))
    assert back.layers == spec.layers and back.width == spec.width and back.vocab == spec.vocab
    assert back.rms_eps == spec.rms_eps and back.embed_scale == spec.embed_scale
    assert back.layers[4].window == 0 and back.layers[4].ff is None and back.layers[2].kv_from == 0
    with pytest.raises(ValueError):
        R.RamopelSpec.from_config(cfg, None)                         # no tensor shapes, no decay rank
    with pytest.raises(ValueError):
        R.RamopelSpec.from_config({**cfg, "architecture": "Other"}, None)
    loaded = R.load_checkpoint(path)
    assert set(loaded) == set(sd) and all(torch.equal(loaded[k], sd[k]) for k in sd)


def test_resolve_model_picks_the_class_by_config(tmp_path):
    from llmq_b200.model import BUILTIN_SPECS, resolve_model
    spec = small_spec()
    (tmp_path / "config.json").write_text(json.dumps(spec.to_config()))
    R.save_checkpoint(str(tmp_path / "model.safetensors"), checkpoint(spec, 2))
    got, d = resolve_model(str(tmp_path))
    assert isinstance(got, R.RamopelSpec) and got.layers == spec.layers and d == str(tmp_path)
    assert BUILTIN_SPECS["ramopel-1b"].layered and resolve_model("random:ramopel-1b")[1] is None


def test_engine_weights_shapes_and_fusions():
    spec = small_spec()
    sd = checkpoint(spec, 3)
    ew = dict(R.engine_weights(spec, sd))
    W = spec.width
    a0, d1, a2 = spec.layers[0], spec.layers[1], spec.layers[2]
    assert ew["layers.0.mix.down"].shape == (a0.q_rank + a0.kv_rank + a0.rot_dim, W)
    assert ew["layers.2.mix.down"].shape == (a2.q_rank, W) and "layers.2.mix.kv_norm" not in ew
    assert ew["layers.1.mix.proj"].shape == (5 * d1.heads * d1.dim + d1.decay_rank, W)
    # the transposed key up-projection: q . (W_uk c) == (W_uk^T q) . c for every head
    g = torch.Generator().manual_seed(0)
    q = torch.randn(a0.heads, a0.dim, generator=g, dtype=torch.float64)
    c = torch.randn(a0.kv_rank, generator=g, dtype=torch.float64)
    uk = sd["l0.mix.uk"].double().view(a0.heads, a0.dim, a0.kv_rank)
    ukt = ew["layers.0.mix.uk_t"].double().view(a0.heads, a0.kv_rank, a0.dim)
    assert torch.allclose(torch.einsum("hd,hdr,r->h", q, uk, c), torch.einsum("hrd,hd,r->h", ukt, q, c))
    E, F = a0.n_experts, a0.ff_dim
    gu = ew["layers.0.mlp.experts_gate_up"].view(E, 2, F, W)
    assert torch.equal(gu[3, 0], sd["l0.mlp.e3.gate"]) and torch.equal(gu[3, 1], sd["l0.mlp.e3.up"])
    assert torch.equal(ew["layers.0.mlp.experts_down"].view(E, W, F)[4], sd["l0.mlp.e4.down"])
    assert all(t.dim() in (1, 2) for t in ew.values())


def test_oracle_is_causal_and_windowed():
    """the oracle itself: a token never depends on later tokens, and an attention-only model with window w
    forgets a token exactly w places later"""
    spec = small_spec(layers=[attn(window=6, **DENSE)])
    sd = checkpoint(spec, 4)
    cfg = spec.to_config()
    a = tokens(30, spec.vocab, 1)
    b = list(a)
    b[10] = (b[10] + 1) % spec.vocab
    la, lb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    assert torch.equal(la[:10], lb[:10])
    assert not torch.allclose(la[15], lb[15]) and torch.allclose(la[16:], lb[16:], atol=1e-12)
    # the recurrence carries state: cutting the sequence and passing S on is the same as not cutting
    g = torch.Generator().manual_seed(1)
    r, k, v = (torch.randn(12, 8, generator=g, dtype=torch.float64) for _ in range(3))
    w, al = torch.rand(12, 8, generator=g, dtype=torch.float64), torch.rand(12, 8, generator=g, dtype=torch.float64)
    o, S = O.delta_rule_steps(r, k, v, w, al)
    o1, S1 = O.delta_rule_steps(r[:5], k[:5], v[:5], w[:5], al[:5])
    o2, S2 = O.delta_rule_steps(r[5:], k[5:], v[5:], w[5:], al[5:], S1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(S2, S)


def _dry(max_seqs, num_blocks, max_tokens=256):
    lib = L.load()
    cfg = L.EngineConfig(max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens, max_model_len=max_tokens,
                         eos_token_id=-1, policy=1)
    h = C.c_void_p()
    L.check(lib.b200q_engine_create_dryrun(C.byref(cfg), 100, 16, num_blocks, C.byref(h)))
    return lib, h


def _replay(lib, h, entries):
    ids = np.asarray([e[0] for e in entries], dtype=np.int64)
    nt = np.asarray([len(e[1]) for e in entries], dtype=np.int32)
    tk = np.concatenate([np.asarray(e[1], dtype=np.int32) for e in entries])
    nw = np.asarray([len(e[2]) for e in entries], dtype=np.int32)
    w = np.concatenate([np.asarray(e[2], dtype=np.int32) for e in entries] + [np.zeros(1, np.int32)])
    return lib.b200q_engine_step_replay(h, len(entries), ids.ctypes.data, nt.ctypes.data, tk.ctypes.data,
                                        nw.ctypes.data, w.ctypes.data, None)


def test_replayed_steps_reuse_pages_and_slots_dryrun():
    lib, h = _dry(max_seqs=2, num_blocks=4)
    st = L.EngineStats()
    assert _replay(lib, h, [(1, [1] * 20, [19]), (2, [2] * 30, [0, 29])]) == 0       # 2 + 2 pages
    assert _replay(lib, h, [(2, [3], [0])]) == 0                                       # request 1 sits out
    # a third live request has no slot; a step that needs a fifth page is refused and leaves no trace
    assert _replay(lib, h, [(3, [4], [0])]) != 0
    assert _replay(lib, h, [(1, [5] * 13, [])]) != 0                                   # 33 tokens: a third page
    lib.b200q_engine_get_stats(h, C.byref(st))
    assert st.free_blocks == 0 and st.running == 2
    lib.b200q_engine_abort(h, 1)
    assert _replay(lib, h, [(3, [4] * 32, [31]), (2, [6], [0])]) == 0                  # 1's pages and slot, reused
    assert _replay(lib, h, [(2, [7], [0]), (2, [8], [0])]) != 0                        # a request twice in a step
    assert _replay(lib, h, [(2, [100], [0])]) != 0                                     # token id out of range
    assert _replay(lib, h, [(2, [7], [1])]) != 0                                       # wanted place out of range
    lib.b200q_engine_abort(h, 2)
    lib.b200q_engine_abort(h, 3)
    lib.b200q_engine_get_stats(h, C.byref(st))
    assert st.free_blocks == 4 and st.running == 0
    lib.b200q_engine_destroy(h)
