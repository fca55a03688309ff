"""Plain, slow restatement of the Ramopel decoder (test infrastructure only; the product never
imports it).  One function per mechanism, whole sequences at once, no cache, no batching: every
position is recomputed from the tokens, so a fault of the engine's pages, slots, windows or chunking
cannot hide here.

Ramopel = parallel layers  x <- x + mixer(norm1 x) + ff(norm2 x)  over two mixer kinds
(latent attention with a sliding window, optionally reading another layer's cached latents; a
generalized delta-rule recurrence) and two feed-forward kinds (PolyNorm dense; top-k mixture of
clamped gated experts plus a gated shared expert).

`weights` maps the checkpoint's tensor names to torch tensors; `cfg` is the parsed config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def centered_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is an offset from one"""
    return rms_unit(x, eps) * (1.0 + w)


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [..., T, n>=dims]; the first `dims` entries are rotated as pairs (2i, 2i+1) by the angle
    pos * base^(-2i/dims); the rest pass through.  pos [T]."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    f = base ** (-2.0 * i / dims)
    a = pos.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_kv(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """what a latent-attention layer caches: the normed latent c [T, kv_rank] and the shared rotated key
    part [T, rot_dim] (after rotation)"""
    T = h.shape[0]
    R, P = mx["kv_rank"], mx["rot_dim"]
    d = h @ w[pre + "dkv"].T
    c = rms_unit(d[:, :R], eps) * w[pre + "dkv.norm"]
    kr = rotate_pairs(d[:, R:R + P], torch.arange(T), mx["rot"]["base"], mx["rot"]["dims"])
    return c, kr


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict, eps: float,
                     c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    """h [T, width] -> [T, width]; c, kr are the (own or borrowed) cached latents"""
    T = h.shape[0]
    H, D, P, V = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
    cq = rms_unit(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, D + P)
    qn, qr = q[..., :D], q[..., D:]
    qr = rotate_pairs(qr.transpose(0, 1), torch.arange(T), mx["rot"]["base"], mx["rot"]["dims"]).transpose(0, 1)
    kn = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, V)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihp,jp->hij", qr, kr)) * mx["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    size = (mx.get("mask") or {}).get("size", 0)   # no mask entry: every earlier key is seen
    seen = (i - j >= 0) & ((i - j < size) if size else (i - j >= 0))
    s = s.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hij,jhv->ihv", p, v).reshape(T, H * V)
    return o @ w[pre + "o"].T


def general_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict, eps: float) -> torch.Tensor:
    """generalized delta rule, token by token, state [heads, key, value] from zero"""
    T = h.shape[0]
    H, D = mx["heads"], mx["dim"]
    r = (h @ w[pre + "r"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, H, D)
    v = (h @ w[pre + "v"].T).view(T, H, D)
    dec = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"])).view(T, H, D)
    a = torch.sigmoid(h @ w[pre + "a"].T + w[pre + "a.b"]).view(T, H, D)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, D, dtype=h.dtype)
    out = torch.zeros(T, H, D, dtype=h.dtype)
    for t in range(T):
        uS = torch.einsum("hi,hij->hj", u[t], S)
        S = dec[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hij,hi->hj", S, r[t])
    o = rms_unit(out, eps).reshape(T, H * D) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def polynorm_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    z = h @ w[pre + "up"].T
    a, b, c, e = w[pre + "act"].tolist()
    y = a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e
    return y @ w[pre + "down"].T


def clamped_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, limit: float) -> torch.Tensor:
    g = (h @ w[pre + "gate"].T).clamp(max=limit)
    u = (h @ w[pre + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, ml: dict) -> torch.Tensor:
    E, top = ml["router"]["experts"], ml["router"]["top"]
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    gate = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for kk in range(top):
            e = int(idx[t, kk])
            out[t] += gate[t, kk] * clamped_expert(h[t:t + 1], w, f"{pre}e{e}.", ml["expert"]["limit"])[0]
    if ml.get("shared"):
        sg = torch.sigmoid(h @ w[pre + "shared.sg"].T)
        out = out + sg * clamped_expert(h, w, pre + "shared.", ml["shared"]["limit"])
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            keep_layers: bool = False):
    """logits [T, vocab] of one sequence (and, if asked, the residual stream after every layer)"""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    latents: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    stream = []
    for i, lc in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h1 = centered_norm(x, w[pre + "norm1"], eps)
        mx = lc["mixer"]
        if lc["type"] == "latent_attention":
            if mx.get("kv_from") is None:
                latents[i] = latent_kv(h1, w, pre + "mix.", mx, eps)
                c, kr = latents[i]
            else:
                c, kr = latents[mx["kv_from"]]
            m = latent_attention(h1, w, pre + "mix.", mx, eps, c, kr)
        elif lc["type"] == "general_delta":
            m = general_delta(h1, w, pre + "mix.", mx, eps)
        else:
            raise ValueError(lc["type"])
        f = 0.0
        ml = lc.get("mlp")
        if ml:
            h2 = centered_norm(x, w[pre + "norm2"], eps)
            f = polynorm_ff(h2, w, pre + "mlp.", eps) if ml["kind"] == "dense" else moe_ff(h2, w, pre + "mlp.", ml)
        x = x + (m + f)
        if keep_layers:
            stream.append(x.clone())
    logits = centered_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(stream)) if keep_layers else logits


def windowed_attention(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, pos: torch.Tensor,
                       window: int, scale: float) -> torch.Tensor:
    """q [n, H, d] asked at positions pos [n]; keys [L, d], values [L, r] of one sequence (shared by the
    heads).  Position p sees j with 0 <= p - j < window (window 0: every j <= p).  -> [n, H, r]"""
    out = torch.zeros(q.shape[0], q.shape[1], values.shape[1], dtype=q.dtype)
    for i in range(q.shape[0]):
        p = int(pos[i])
        lo = max(0, p - window + 1) if window > 0 else 0
        s = torch.einsum("hd,jd->hj", q[i], keys[lo:p + 1]) * scale
        out[i] = torch.softmax(s, -1) @ values[lo:p + 1]
    return out


def delta_rule_steps(r, k, v, w, a, S0=None):
    """the recurrence alone, one head: r, k, v, w (decay), a (removal) [T, D]; S0 [D, D] or None (zero).
    -> (o [T, D], S_T)"""
    T, D = k.shape
    S = torch.zeros(D, D, dtype=k.dtype) if S0 is None else S0.clone()
    o = torch.zeros(T, D, dtype=k.dtype)
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum() + 1e-6)
        S = w[t][:, None] * S - (a[t] * u)[:, None] * (u @ S)[None, :] + k[t][:, None] * v[t][None, :]
        o[t] = S.T @ r[t]
    return o, S


def greedy(cfg: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int, dtype=torch.float64) -> List[int]:
    """greedy continuation, every step recomputed from the tokens"""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks, dtype)[-1].argmax()))
    return toks[len(prompt):]
