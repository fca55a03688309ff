"""Host side of the Noridra decoder: reading its config.json, mapping its checkpoint to the engine's
layered-model weights, and drawing random checkpoints for tests and benchmarks.

Noridra is a stack of post-norm layers over an fp32 residual stream,

    x <- N1(alpha x + s1 * mixer(x + conv1 x))        x <- N2(alpha x + s2 * ff(x + conv2 x))

with grouped RMS norms N, per-channel layer scales s, and per-channel causal input convolutions whose last
inputs travel with the sequence.  Token and learned position embeddings are summed.  Mixers: a gated delta
rule (short convolutions on q, k, v; unit-norm q and k; per-head decay and write strength), chunked
grouped-query attention whose values are its raw keys (per-head norms, soft cap, logarithmic distance
penalty, sink softmax, sigmoid output gate), and a selective scan.  The feed-forward is a top-k mixture of
gated experts routed by sigmoid scores that scale the expert's input.  Every size comes from config.json;
the native side takes one `b200q_layer_desc` per layer (`b200q_model_create_layered`), so other layered
designs can reuse the same mixers with other constants.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import lib as L
from .ramopel import checkpoint_shapes, load_checkpoint, save_checkpoint  # noqa: F401  (one file format)

ARCHITECTURE = "Noridra"
_MIXERS = {"delta": L.MIXER_GATED_DELTA, "attention": L.MIXER_CHUNK_ATTN, "mamba1": L.MIXER_SELECTIVE_SCAN}


@dataclass
class NoridraLayer:
    mixer: str                       # "delta" | "attention" | "mamba1"
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0                     # per-head size of q and k
    vdim: int = 0                    # per-head size of v (attention: the values are the keys, vdim == dim)
    conv: int = 0                    # delta / mamba1: taps of the mixer's short convolution
    scale: float = 1.0               # attention: score scale
    softcap: float = 0.0             # attention: 0 = off
    chunk: int = 0                   # attention: positions per chunk, 0 = plain causal
    inner: int = 0                   # mamba1: channels
    state: int = 0                   # mamba1: state size per channel
    dt_rank: int = 0                 # mamba1: rank of the step-size projection
    ff: Optional[str] = None         # None | "moe"
    ff_dim: int = 0
    n_experts: int = 0
    top_k: int = 0

    def desc(self) -> L.LayerDesc:
        return L.LayerDesc(
            mixer=_MIXERS[self.mixer], heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim,
            conv_taps=self.conv, attn_scale=self.scale, softcap=self.softcap, chunk=self.chunk, inner=self.inner,
            state_dim=self.state, dt_rank=self.dt_rank, kv_from=-1,
            ff=L.FF_MOE_SIGMOID if self.ff == "moe" else L.FF_NONE, ff_dim=self.ff_dim, n_experts=self.n_experts,
            top_k=self.top_k)


@dataclass
class NoridraSpec:
    """What `NativeModel` needs to know about a Noridra checkpoint (the counterpart of `ModelSpec`)."""
    width: int
    vocab: int
    layers: List[NoridraLayer]
    rms_eps: float = 1e-6
    norm_groups: int = 1
    alpha: float = 1.0
    canon_taps: int = 0
    max_position_embeddings: int = 2048      # rows of the learned position table
    name: str = "noridra"
    eos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    arch: str = "noridra"
    layered: bool = field(default=True, repr=False)

    @property
    def hidden(self) -> int:
        return self.width

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def config_extras(self) -> dict:
        """the fields of b200q_model_config that describe this design's layer form"""
        return dict(arch=L.ARCH_NORIDRA, layer_form=L.FORM_POSTNORM, norm_groups=self.norm_groups,
                    residual_alpha=self.alpha, input_taps=self.canon_taps, learned_pos=1, embed_scale=0.0)

    @staticmethod
    def from_config(cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None,
                    name: str = "noridra") -> "NoridraSpec":
        if cfg.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture={cfg.get('architecture')!r}")
        layers: List[NoridraLayer] = []
        for i, lc in enumerate(cfg["layers"]):
            mx, kind = lc["mixer"], lc["type"]
            if kind == "delta":
                ly = NoridraLayer(mixer=kind, heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])),
                                  dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])), conv=int(mx["conv"]))
            elif kind == "attention":
                ly = NoridraLayer(mixer=kind, heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])),
                                  dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])), scale=float(mx["scale"]),
                                  softcap=float(mx.get("softcap") or 0.0),
                                  chunk=int((mx.get("mask") or {}).get("size") or 0))
                if ly.vdim != ly.dim:
                    raise ValueError(f"layer {i}: the values are the keys, so vdim ({ly.vdim}) must equal dim ({ly.dim})")
            elif kind == "mamba1":
                ly = NoridraLayer(mixer=kind, inner=int(mx["inner"]), state=int(mx["state"]), dt_rank=int(mx["dt_rank"]),
                                  conv=int(mx["conv"]))
            else:
                raise ValueError(f"layer {i}: unknown layer type {kind!r}")
            if ly.mixer != "mamba1" and ly.heads % ly.kv_heads:
                raise ValueError(f"layer {i}: kv_heads ({ly.kv_heads}) must divide heads ({ly.heads})")
            ml = lc.get("mlp")
            if ml:
                if ml.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {ml['kind']!r}")
                ly.ff, ly.ff_dim = "moe", int(ml["expert"]["ff"])
                ly.n_experts, ly.top_k = int(ml["router"]["experts"]), int(ml["router"]["top"])
            layers.append(ly)
        norm = cfg.get("norm") or {}
        return NoridraSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers,
                           rms_eps=float(norm.get("eps", 1e-6)), norm_groups=int(norm.get("groups", 1)),
                           alpha=float(cfg.get("postln_alpha", 1.0)), canon_taps=int((cfg.get("canon") or {}).get("taps", 0)),
                           max_position_embeddings=int(cfg["max_positions"]), name=name)

    def to_config(self) -> dict:
        out = []
        for ly in self.layers:
            if ly.mixer == "delta":
                mx = {"heads": ly.heads, "kv_heads": ly.kv_heads, "dim": ly.dim, "vdim": ly.vdim, "conv": ly.conv}
            elif ly.mixer == "attention":
                mx = {"heads": ly.heads, "kv_heads": ly.kv_heads, "dim": ly.dim, "vdim": ly.vdim, "scale": ly.scale}
                if ly.softcap:
                    mx["softcap"] = ly.softcap
                if ly.chunk:
                    mx["mask"] = {"size": ly.chunk}
            else:
                mx = {"inner": ly.inner, "state": ly.state, "dt_rank": ly.dt_rank, "conv": ly.conv}
            ml = None
            if ly.ff == "moe":
                ml = {"kind": "moe", "expert": {"ff": ly.ff_dim}, "router": {"experts": ly.n_experts, "top": ly.top_k}}
            out.append({"type": ly.mixer, "mixer": mx, "mlp": ml})
        return {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab,
                "norm": {"eps": self.rms_eps, "groups": self.norm_groups}, "postln_alpha": self.alpha,
                "canon": {"taps": self.canon_taps}, "max_positions": self.max_position_embeddings, "layers": out}

    def engine_weights(self, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
        return engine_weights(self, sd)

    def random_checkpoint(self, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
        return random_checkpoint(self, seed, device)

    def weight_bytes_per_token(self, esize: int = 2, batch: int = 1) -> int:
        """matrix bytes one decode step of `batch` tokens touches (a routed layer reads at most
        min(experts, batch * top_k) of its experts; embedding and position rows are read by row)"""
        W, n = self.width, self.vocab * self.width
        for ly in self.layers:
            if ly.mixer == "delta":
                gd, hv = ly.kv_heads * ly.dim, ly.heads * ly.vdim
                n += W * (2 * gd + 2 * hv + 2 * ly.heads) + W * hv
            elif ly.mixer == "attention":
                hd = ly.heads * ly.dim
                n += W * (2 * hd + ly.kv_heads * ly.dim) + W * hd
            else:
                n += W * 2 * ly.inner + ly.inner * (ly.dt_rank + 2 * ly.state) + ly.inner * ly.dt_rank + W * ly.inner
            if ly.ff == "moe":
                n += W * ly.n_experts + 3 * W * ly.ff_dim * min(ly.n_experts, batch * ly.top_k)
        return n * esize


# ---- checkpoint names -> engine names --------------------------------------------------------------
def engine_weights(spec: NoridraSpec, sd: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
    """Checkpoint tensors -> the layered engine's weights.  2-D results are matrices (bound in the model's
    dtype); 1-D results are vectors, constants and convolution taps (bound as fp32 rows, a [C, taps] table
    flattened row by row).  Fusions: the token projections of a mixer that read the same input become one
    matrix (delta: q, k, v, gate and, apart, the two per-head rows beta / decay; attention: q, k, gate),
    the three short convolutions of a delta layer become one table over the channels q | k | v, gate and up
    of every expert are stacked."""
    yield "embed", sd["embed"]
    yield "pos", sd["pos"]
    yield "final_norm", sd["final.norm"]
    yield "lm_head", sd["head"]
    for i, ly in enumerate(spec.layers):
        p, o = f"l{i}.", f"layers.{i}."
        yield o + "norm1", sd[p + "norm1"]
        yield o + "ls1", sd[p + "ls1"]
        if spec.canon_taps:
            yield o + "canon1", sd[p + "canon1"].reshape(-1)
        if ly.ff is not None:
            yield o + "norm2", sd[p + "norm2"]
            yield o + "ls2", sd[p + "ls2"]
            if spec.canon_taps:
                yield o + "canon2", sd[p + "canon2"].reshape(-1)
        m = p + "mix."
        if ly.mixer == "delta":
            yield o + "mix.proj", torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "g"]], 0)
            yield o + "mix.ba", torch.cat([sd[m + "b"], sd[m + "a"]], 0)
            yield o + "mix.conv", torch.cat([sd[m + "q.conv"], sd[m + "k.conv"], sd[m + "v.conv"]], 0).reshape(-1)
            yield o + "mix.a_log", sd[m + "A_log"]
            yield o + "mix.dt_bias", sd[m + "dt_bias"]
            yield o + "mix.out_norm", sd[m + "norm"]
            yield o + "mix.o", sd[m + "o"]
        elif ly.mixer == "attention":
            yield o + "mix.proj", torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "g"]], 0)
            yield o + "mix.q_norm", sd[m + "q.norm"]
            yield o + "mix.k_norm", sd[m + "k.norm"]
            yield o + "mix.r1", sd[m + "r1"]
            yield o + "mix.r2", sd[m + "r2"]
            yield o + "mix.o", sd[m + "o"]
        else:
            yield o + "mix.proj", sd[m + "in"]
            yield o + "mix.conv", sd[m + "conv"].reshape(-1)
            yield o + "mix.conv_b", sd[m + "conv.b"]
            xw = sd[m + "x"]                       # [dt | B | C] rows, padded with zero rows to a multiple of 64
            pad = -xw.shape[0] % 64
            yield o + "mix.x", (torch.cat([xw, xw.new_zeros(pad, xw.shape[1])], 0) if pad else xw)
            yield o + "mix.dt", sd[m + "dt"]
            yield o + "mix.dt_b", sd[m + "dt.b"]
            yield o + "mix.a_log", sd[m + "A_log"].reshape(-1)
            yield o + "mix.d", sd[m + "D"]
            yield o + "mix.o", sd[m + "o"]
        if ly.ff == "moe":
            f = p + "mlp."
            yield o + "mlp.router", sd[f + "router"]
            yield o + "mlp.experts_gate_up", torch.cat(
                [t for e in range(ly.n_experts) for t in (sd[f"{f}e{e}.gate"], sd[f"{f}e{e}.up"])], 0)
            yield o + "mlp.experts_down", torch.cat([sd[f"{f}e{e}.down"] for e in range(ly.n_experts)], 0)


def random_checkpoint(spec: NoridraSpec, seed: int = 0, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """A random checkpoint in the checkpoint's own names.  Matrices are Normal(0, 1/sqrt(fan_in)); norm
    weights, layer scales, convolution taps, decay constants and distance-penalty constants are non-trivial
    values so that none of them is silently ignored."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = spec.width

    def mat(r, c, s=None):
        s = s if s is not None else c ** -0.5
        return (torch.randn(r, c, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    def vec(n, mean=0.0, s=0.1):
        return (mean + torch.randn(n, generator=g, device=device, dtype=torch.float32) * s).to(dtype)

    def uni(n, lo, hi):
        return (lo + (hi - lo) * torch.rand(n, generator=g, device=device, dtype=torch.float32)).to(dtype)

    sd = {"embed": mat(spec.vocab, W, 1.0), "pos": mat(spec.max_position_embeddings, W, 0.5),
          "final.norm": vec(W, 1.0), "head": mat(spec.vocab, W)}
    for i, ly in enumerate(spec.layers):
        p = f"l{i}."
        subs = ("1", "2") if ly.ff is not None else ("1",)
        for s in subs:
            sd[p + "norm" + s] = vec(W, 1.0)
            sd[p + "ls" + s] = vec(W, 1.0, 0.25)
            if spec.canon_taps:
                sd[p + "canon" + s] = mat(W, spec.canon_taps, 0.3)
        m = p + "mix."
        if ly.mixer == "delta":
            gd, hv = ly.kv_heads * ly.dim, ly.heads * ly.vdim
            sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "g"] = mat(gd, W), mat(gd, W), mat(hv, W), mat(hv, W)
            for n, c in (("q", gd), ("k", gd), ("v", hv)):
                sd[m + n + ".conv"] = mat(c, ly.conv, 0.5)
            sd[m + "b"], sd[m + "a"] = mat(ly.heads, W), mat(ly.heads, W)
            sd[m + "A_log"] = uni(ly.heads, -2.0, 0.5)
            sd[m + "dt_bias"] = vec(ly.heads, 0.0, 0.5)
            sd[m + "norm"] = vec(ly.vdim, 1.0)
            sd[m + "o"] = mat(W, hv)
        elif ly.mixer == "attention":
            hd = ly.heads * ly.dim
            sd[m + "q"], sd[m + "k"], sd[m + "g"] = mat(hd, W), mat(ly.kv_heads * ly.dim, W), mat(hd, W)
            sd[m + "q.norm"], sd[m + "k.norm"] = vec(ly.dim, 1.0), vec(ly.dim, 1.0)
            sd[m + "r1"], sd[m + "r2"] = uni(ly.heads, 0.1, 1.0), uni(ly.heads, 0.05, 2.0)
            sd[m + "o"] = mat(W, hd)
        else:
            sd[m + "in"] = mat(2 * ly.inner, W)
            sd[m + "conv"], sd[m + "conv.b"] = mat(ly.inner, ly.conv, 0.5), vec(ly.inner)
            sd[m + "x"] = mat(ly.dt_rank + 2 * ly.state, ly.inner)
            sd[m + "dt"], sd[m + "dt.b"] = mat(ly.inner, ly.dt_rank), vec(ly.inner, -1.0, 0.5)
            sd[m + "A_log"] = uni(ly.inner * ly.state, -1.0, 1.5).reshape(ly.inner, ly.state)
            sd[m + "D"] = vec(ly.inner, 1.0)
            sd[m + "o"] = mat(W, ly.inner)
        if ly.ff == "moe":
            f = p + "mlp."
            sd[f + "router"] = mat(ly.n_experts, W, 2.0 * W ** -0.5)
            for e in range(ly.n_experts):
                sd[f"{f}e{e}.gate"] = mat(ly.ff_dim, W)
                sd[f"{f}e{e}.up"] = mat(ly.ff_dim, W)
                sd[f"{f}e{e}.down"] = mat(W, ly.ff_dim)
    return sd


def _cycle(width: int, vocab: int, n_layers: int, heads: int, kv_heads: int, dim: int, experts: int, top: int,
           ff: int, name: str) -> NoridraSpec:
    """layers in the order delta, attention, mamba1, delta, ... with a routed feed-forward in every layer"""
    layers: List[NoridraLayer] = []
    for i in range(n_layers):
        kind = ("delta", "attention", "mamba1", "delta")[i % 4]
        moe = dict(ff="moe", ff_dim=ff, n_experts=experts, top_k=top)
        if kind == "delta":
            layers.append(NoridraLayer(mixer="delta", heads=heads, kv_heads=heads, dim=dim, vdim=dim, conv=4, **moe))
        elif kind == "attention":
            layers.append(NoridraLayer(mixer="attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim,
                                       scale=dim ** -0.5, softcap=50.0, chunk=2048, **moe))
        else:
            layers.append(NoridraLayer(mixer="mamba1", inner=2 * width, state=16, dt_rank=width // 16, conv=4, **moe))
    return NoridraSpec(width=width, vocab=vocab, layers=layers, rms_eps=1e-6, norm_groups=4, alpha=2.0, canon_taps=4,
                       max_position_embeddings=8192, name=name)


# sizes that resemble a real model's layers (random weights; `random:<name>` as a model name)
BUILTIN_SPECS = {
    "noridra-1b": _cycle(2048, 32768, 16, 16, 4, 128, 16, 4, 1024, "noridra-1b"),
    "noridra-3b": _cycle(3072, 32768, 24, 24, 8, 128, 32, 6, 1536, "noridra-3b"),
}
