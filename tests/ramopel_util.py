"""Shared helpers of the Ramopel tests: small configurations with sizes that differ from one another
(heads*dim != width, rot_dim != dim, vdim != dim, several head groups, experts with and without a shared
one, a layer without feed-forward), random checkpoints, and error measures."""
import numpy as np
import torch

from llmq_b200.ramopel import RamopelLayer, RamopelSpec, random_checkpoint


def attn(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=48, window=20, kv_from=-1, base=10000.0, scale=0.2,
         **ff):
    return RamopelLayer(mixer="latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank,
                        kv_rank=kv_rank, kv_from=kv_from, window=window, rot_dims=rot_dim, rot_base=base,
                        attn_scale=scale, **ff)


def delta(heads=2, dim=32, rank=8, **ff):
    return RamopelLayer(mixer="general_delta", heads=heads, dim=dim, decay_rank=rank, **ff)


DENSE = dict(ff="dense", ff_dim=72)
MOE = dict(ff="moe", ff_dim=40, n_experts=6, top_k=2, expert_limit=1.5, shared_dim=56, shared_limit=0.75)
MOE_PLAIN = dict(ff="moe", ff_dim=24, n_experts=5, top_k=1, expert_limit=3.0)


def small_spec(width=96, vocab=211, layers=None, eps=1e-5, embed_scale=0.75):
    layers = layers or [
        attn(**MOE),                                              # owns its latents
        delta(**DENSE),
        attn(heads=9, dim=8, vdim=16, window=7, kv_from=0, scale=0.35, **DENSE),   # reads layer 0's, two head groups
        delta(heads=3, dim=16, rank=5, **MOE_PLAIN),
        attn(heads=2, dim=24, rot_dim=16, vdim=8, q_rank=24, kv_rank=32, window=0, base=500.0),  # no window, no ff
    ]
    return RamopelSpec(width=width, vocab=vocab, layers=layers, rms_eps=eps, embed_scale=embed_scale)


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
