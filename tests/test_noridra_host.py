"""CPU tests of the Noridra host code: the config reader, the registry, the mapping of checkpoint tensors to
engine weights, and the oracle's own consistency (causality, chunk confinement, the sink, convolutions that
start from zeros, recurrences that can be cut and continued)."""
import json

import pytest
import torch

from llmq_b200 import lib as L
from llmq_b200 import noridra as N
from oracle import noridra as O
from tests.noridra_util import MOE, attn, checkpoint, delta, scan, small_spec, tokens


def test_config_round_trip(tmp_path):
    spec = small_spec()
    cfg = json.loads(json.dumps(spec.to_config()))
    back = N.NoridraSpec.from_config(cfg)
    assert back.layers == spec.layers and back.width == spec.width and back.vocab == spec.vocab
    assert (back.rms_eps, back.norm_groups, back.alpha, back.canon_taps) == (1e-5, 3, 1.7, 3)
    assert back.layers[2].ff is None and back.layers[3].chunk == 0 and back.layers[3].softcap == 0.0
    assert back.max_position_embeddings == spec.max_position_embeddings
    with pytest.raises(ValueError):
        N.NoridraSpec.from_config({**cfg, "architecture": "Other"})
    bad = json.loads(json.dumps(cfg))
    bad["layers"][1]["mixer"]["vdim"] = 8                              # the values are the keys
    with pytest.raises(ValueError):
        N.NoridraSpec.from_config(bad)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][0]["type"] = "unknown"
    with pytest.raises(ValueError):
        N.NoridraSpec.from_config(bad)
    ex = spec.config_extras()
    assert ex["arch"] == L.ARCH_NORIDRA and ex["layer_form"] == L.FORM_POSTNORM and ex["learned_pos"] == 1
    d0, a1, s2 = (ly.desc() for ly in spec.layers[:3])
    assert (d0.mixer, d0.kv_heads, d0.vdim, d0.conv_taps, d0.top_k) == (L.MIXER_GATED_DELTA, 2, 24, 3, 2)
    assert (a1.mixer, a1.chunk, a1.ff) == (L.MIXER_CHUNK_ATTN, 20, L.FF_MOE_SIGMOID)
    assert (s2.mixer, s2.inner, s2.state_dim, s2.dt_rank, s2.ff) == (L.MIXER_SELECTIVE_SCAN, 80, 12, 5, L.FF_NONE)


def test_resolve_model_picks_the_class_by_config(tmp_path):
    from llmq_b200.model import BUILTIN_SPECS, resolve_model
    spec = small_spec()
    sd = checkpoint(spec, 2)
    (tmp_path / "config.json").write_text(json.dumps(spec.to_config()))
    N.save_checkpoint(str(tmp_path / "model.safetensors"), sd)
    got, d = resolve_model(str(tmp_path))
    assert isinstance(got, N.NoridraSpec) and got.layers == spec.layers and d == str(tmp_path)
    assert BUILTIN_SPECS["noridra-1b"].layered and resolve_model("random:noridra-1b")[1] is None
    loaded = N.load_checkpoint(str(tmp_path / "model.safetensors"))
    assert set(loaded) == set(sd) and all(torch.equal(loaded[k], sd[k]) for k in sd)


def test_engine_weights_shapes_and_fusions():
    spec = small_spec()
    sd = checkpoint(spec, 3)
    ew = dict(spec.engine_weights(sd))
    W = spec.width
    d0, a1, s2 = spec.layers[0], spec.layers[1], spec.layers[2]
    gd, hv = d0.kv_heads * d0.dim, d0.heads * d0.vdim
    assert ew["layers.0.mix.proj"].shape == (2 * gd + 2 * hv, W)
    assert torch.equal(ew["layers.0.mix.proj"][gd:2 * gd], sd["l0.mix.k"])
    assert torch.equal(ew["layers.0.mix.proj"][2 * gd + hv:], sd["l0.mix.g"])
    assert torch.equal(ew["layers.0.mix.ba"][d0.heads:], sd["l0.mix.a"])
    conv = ew["layers.0.mix.conv"].view(2 * gd + hv, d0.conv)
    assert torch.equal(conv[gd:2 * gd], sd["l0.mix.k.conv"]) and torch.equal(conv[2 * gd:], sd["l0.mix.v.conv"])
    hd = a1.heads * a1.dim
    assert ew["layers.1.mix.proj"].shape == (2 * hd + a1.kv_heads * a1.dim, W)
    assert torch.equal(ew["layers.1.mix.proj"][hd + a1.kv_heads * a1.dim:], sd["l1.mix.g"])
    assert ew["layers.2.mix.a_log"].shape == (s2.inner * s2.state,) and "layers.2.norm2" not in ew
    assert ew["layers.0.canon1"].shape == (W * spec.canon_taps,) and ew["pos"].shape == (spec.max_position_embeddings, W)
    E, F = d0.n_experts, d0.ff_dim
    gu = ew["layers.0.mlp.experts_gate_up"].view(E, 2, F, W)
    assert torch.equal(gu[3, 0], sd["l0.mlp.e3.gate"]) and torch.equal(gu[3, 1], sd["l0.mlp.e3.up"])
    assert torch.equal(ew["layers.0.mlp.experts_down"].view(E, W, F)[4], sd["l0.mlp.e4.down"])
    assert all(t.dim() in (1, 2) for t in ew.values())


def test_oracle_is_causal_and_confined_to_chunks():
    """a token never depends on later tokens; an attention-only model without input convolutions sees nothing
    of an earlier chunk"""
    spec = small_spec(layers=[attn(chunk=8, **MOE)], taps=1)
    sd = checkpoint(spec, 4)
    sd["l0.canon1"].zero_()
    sd["l0.canon2"].zero_()
    cfg = spec.to_config()
    a = tokens(30, spec.vocab, 1)
    b = list(a)
    b[10] = (b[10] + 1) % spec.vocab
    la, lb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    assert torch.equal(la[:10], lb[:10])
    assert not torch.allclose(la[15], lb[15]) and torch.allclose(la[16:], lb[16:], atol=1e-12)
    # with every mixer in the stack, a change is never seen before its place
    spec = small_spec()
    sd, cfg = checkpoint(spec, 5), spec.to_config()
    la, lb = O.forward(cfg, sd, a), O.forward(cfg, sd, b)
    assert torch.equal(la[:10], lb[:10]) and not torch.allclose(la[29], lb[29])


def test_oracle_sink_and_convolution_start():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(5, 2, 4, generator=g, dtype=torch.float64), torch.randn(5, 2, 4, generator=g, dtype=torch.float64)
    z = torch.zeros(2, dtype=torch.float64)
    out = O.sink_attention(q, k, k, z, z, 1.0, 0.0, 0)
    s = (q[0, 0] * k[0, 0]).sum()
    assert torch.allclose(out[0, 0], torch.exp(s) / (1 + torch.exp(s)) * k[0, 0])       # one key and the sink
    x, w = torch.randn(6, 3, generator=g, dtype=torch.float64), torch.randn(3, 4, generator=g, dtype=torch.float64)
    y = O.causal_conv(x, w)
    assert torch.allclose(y[0], w[:, 3] * x[0]) and torch.allclose(y[1], w[:, 3] * x[1] + w[:, 2] * x[0])
    assert torch.allclose(y[5], (w.T * x[2:6]).sum(0))


def test_oracle_norm_groups_and_expert_input_scaling():
    g = torch.Generator().manual_seed(1)
    x, w = torch.randn(4, 12, generator=g, dtype=torch.float64), torch.randn(12, generator=g, dtype=torch.float64)
    y = O.group_norm(x, w, 3, 1e-6)
    assert torch.allclose(y[:, 4:8], x[:, 4:8] / torch.sqrt((x[:, 4:8] ** 2).mean(-1, keepdim=True) + 1e-6) * w[4:8])
    # one expert, top 1: out = expert(s * h) with s the sigmoid score, not s * expert(h)
    W_, F_ = 6, 5
    ws = {"m.router": torch.randn(1, W_, generator=g, dtype=torch.float64),
          "m.e0.gate": torch.randn(F_, W_, generator=g, dtype=torch.float64),
          "m.e0.up": torch.randn(F_, W_, generator=g, dtype=torch.float64),
          "m.e0.down": torch.randn(W_, F_, generator=g, dtype=torch.float64)}
    h = torch.randn(3, W_, generator=g, dtype=torch.float64)
    out = O.experts(h, ws, "m.", {"router": {"top": 1}})
    hin = torch.sigmoid(h @ ws["m.router"].T) * h
    want = (torch.nn.functional.silu(hin @ ws["m.e0.gate"].T) * (hin @ ws["m.e0.up"].T)) @ ws["m.e0.down"].T
    assert torch.allclose(out, want)
