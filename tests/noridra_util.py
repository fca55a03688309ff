"""Shared helpers of the Noridra tests: small configurations whose sizes differ from one another (key heads
fewer than heads, value size unlike key size, convolutions with other tap counts than the input
convolutions, several norm groups, several experts per token, a layer without feed-forward, attention with
and without chunks and soft cap), random checkpoints, and error measures."""
import numpy as np
import torch

from llmq_b200.noridra import NoridraLayer, NoridraSpec, random_checkpoint

MOE = dict(ff="moe", ff_dim=40, n_experts=6, top_k=2)
MOE_ALL = dict(ff="moe", ff_dim=24, n_experts=3, top_k=3)
MOE_ONE = dict(ff="moe", ff_dim=56, n_experts=5, top_k=1)


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, **ff):
    return NoridraLayer(mixer="delta", heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, **ff)


def attn(heads=6, kv_heads=2, dim=24, scale=0.3, softcap=12.0, chunk=20, **ff):
    return NoridraLayer(mixer="attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale,
                        softcap=softcap, chunk=chunk, **ff)


def scan(inner=80, state=12, dt_rank=5, conv=5, **ff):
    return NoridraLayer(mixer="mamba1", inner=inner, state=state, dt_rank=dt_rank, conv=conv, **ff)


def small_spec(width=96, vocab=211, layers=None, eps=1e-5, groups=3, alpha=1.7, taps=3, max_pos=512):
    layers = layers or [
        delta(**MOE),
        attn(**MOE_ONE),                                            # chunks of 20: neither a page nor a tile
        scan(),                                                     # no feed-forward
        attn(heads=3, kv_heads=3, dim=40, softcap=0.0, chunk=0, scale=0.15, **MOE_ALL),   # plain causal, uncapped
        delta(heads=2, kv_heads=2, dim=40, vdim=8, conv=2, **MOE),
        scan(inner=136, state=20, dt_rank=3, conv=2, **MOE_ONE),
    ]
    return NoridraSpec(width=width, vocab=vocab, layers=layers, rms_eps=eps, norm_groups=groups, alpha=alpha,
                       canon_taps=taps, max_position_embeddings=max_pos)


def checkpoint(spec, seed=0):
    """random bf16-representable weights (so the fp32 engine and the fp64 oracle read the same numbers)"""
    return random_checkpoint(spec, seed=seed, device="cpu")


def rel_err(got, want):
    """rms of the difference over the rms of the expected rows, worst row"""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    num = np.sqrt(((got - want) ** 2).mean(-1))
    den = np.sqrt((want ** 2).mean(-1)) + 1e-30
    return float((num / den).max())


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
