"""Plain, slow restatement of the Noridra decoder (test infrastructure only; the product never imports
it).  One function per mechanism, whole sequences at once, no cache, no state slots, no batching: every
position is recomputed from the tokens, so a fault of the engine's pages, slots, chunk borders or
portion handling cannot hide here.

Noridra = post-norm layers over an fp32 residual stream x [T, width]:

    x <- N1(alpha x + s1 * mixer(x + conv1 x))        x <- N2(alpha x + s2 * ff(x + conv2 x))

with N a grouped RMS norm, s1 / s2 per-channel layer scales, conv a per-channel causal convolution over
time, three mixer kinds (gated delta rule, chunked attention whose values are its keys, selective scan)
and a top-k mixture of gated experts whose routing weight scales the expert's input.

`w` maps the checkpoint's tensor names to torch tensors (any float dtype; everything is computed in the
dtype of `dtype`), `cfg` is the parsed config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def group_norm(x: torch.Tensor, wt: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """the last axis is cut into `groups` equal consecutive parts; each is divided by its own
    sqrt(mean(part^2) + eps); the whole is multiplied by wt"""
    sh = x.shape
    p = x.reshape(*sh[:-1], groups, sh[-1] // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(sh) * wt


def causal_conv(x: torch.Tensor, wt: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], wt [C, taps]; y_t = sum_j wt[:, j] x_(t - taps + 1 + j), zeros before the start"""
    T, C = x.shape
    taps = wt.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j:j + T] * wt[:, j]
    if bias is not None:
        y = y + bias
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def gated_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict, eps: float) -> torch.Tensor:
    """h [T, width] -> [T, width].  Per head a state S [dim, vdim]:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q"""
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = F.silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).reshape(T, G, D)
    k = F.silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).reshape(T, G, D)
    v = F.silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).reshape(T, H, V)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[pre + "b"].T)                                        # [T, H]
    g = torch.exp(-torch.exp(w[pre + "A_log"]) * F.softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    gate = F.silu(h @ w[pre + "g"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    rep = H // G
    for hd in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        kh, qh = k[:, hd // rep], q[:, hd // rep]
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kh[t])
            S = S + torch.outer(kh[t], u)
            out[t, hd] = S.T @ qh[t]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w[pre + "norm"] * gate
    return out.reshape(T, H * V) @ w[pre + "o"].T


def sink_attention(qn: torch.Tensor, kn: torch.Tensor, val: torch.Tensor, r1: torch.Tensor, r2: torch.Tensor,
                   scale: float, cap: float, size: int) -> torch.Tensor:
    """qn [T, H, D] and kn [T, G, D] normed queries / keys, val [T, G, D] values -> [T, H, D].  Scores are
    scaled, soft-capped (cap 0: not), lose r1 ln(1 + r2 (i - j)), see j <= i of the same chunk of `size`
    positions (0: all), and the softmax carries one silent extra term of score zero in its denominator"""
    T, H, _ = qn.shape
    rep = H // kn.shape[1]
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).clamp(min=0).to(qn.dtype)
    seen = pos[None, :] <= pos[:, None]
    if size:
        seen = seen & ((pos[:, None] // size) == (pos[None, :] // size))
    out = torch.zeros_like(qn)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd // rep].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s - r1[hd] * torch.log1p(r2[hd] * dist)
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(-1, keepdim=True).values.clamp(min=0.0)
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(-1, keepdim=True))
        out[:, hd] = p @ val[:, hd // rep]
    return out


def chunk_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict, eps: float) -> torch.Tensor:
    """grouped-query attention whose values are the projected keys (before their norm), with a sigmoid
    output gate"""
    T = h.shape[0]
    H, G, D = mx["heads"], mx["kv_heads"], mx["dim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, D)
    kv = (h @ w[pre + "k"].T).reshape(T, G, D)
    qn = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * w[pre + "q.norm"]
    kn = kv / torch.sqrt((kv * kv).mean(-1, keepdim=True) + eps) * w[pre + "k.norm"]
    out = sink_attention(qn, kn, kv, w[pre + "r1"], w[pre + "r2"], mx["scale"], mx.get("softcap") or 0.0,
                         (mx.get("mask") or {}).get("size") or 0)
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * D) * gate) @ w[pre + "o"].T


def selective_scan(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mx: dict) -> torch.Tensor:
    T = h.shape[0]
    I, N, R = mx["inner"], mx["state"], mx["dt_rank"]
    xz = h @ w[pre + "in"].T
    x, z = xz[:, :I], xz[:, I:]
    x = F.silu(causal_conv(x, w[pre + "conv"], w[pre + "conv.b"]))
    p = x @ w[pre + "x"].T
    dt = F.softplus(p[:, :R] @ w[pre + "dt"].T + w[pre + "dt.b"])                  # [T, I]
    B, Cm = p[:, R:R + N], p[:, R + N:R + 2 * N]
    A = -torch.exp(w[pre + "A_log"])                                               # [I, N]
    S = torch.zeros(I, N, dtype=h.dtype)
    y = torch.zeros(T, I, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + w[pre + "D"] * x[t]
    return (y * F.silu(z)) @ w[pre + "o"].T


def experts(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, ml: dict) -> torch.Tensor:
    """sigmoid router, the `top` largest scores (ties: lowest index), weights not renormalised and applied
    to the expert's INPUT"""
    T = h.shape[0]
    top = ml["router"]["top"]
    s = torch.sigmoid(h @ w[pre + "router"].T)
    out = torch.zeros(T, w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(T):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            hin = s[t, e] * h[t]
            p = f"{pre}e{e}."
            out[t] += (F.silu(hin @ w[p + "gate"].T) * (hin @ w[p + "up"].T)) @ w[p + "down"].T
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None,
            n_layers: Optional[int] = None) -> torch.Tensor:
    """logits [T, vocab]; layers_out (a list) receives the residual stream after every layer"""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    eps, groups, alpha = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["postln_alpha"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.shape[0]
    x = w["embed"][ids] + w["pos"][:T]
    for i, lc in enumerate(cfg["layers"][:n_layers]):
        p = f"l{i}."
        hin = x + causal_conv(x, w[p + "canon1"])
        if lc["type"] == "delta":
            m = gated_delta(hin, w, p + "mix.", lc["mixer"], eps)
        elif lc["type"] == "attention":
            m = chunk_attention(hin, w, p + "mix.", lc["mixer"], eps)
        elif lc["type"] == "mamba1":
            m = selective_scan(hin, w, p + "mix.", lc["mixer"])
        else:
            raise ValueError(lc["type"])
        x = group_norm(alpha * x + w[p + "ls1"] * m, w[p + "norm1"], groups, eps)
        if lc.get("mlp"):
            hin = x + causal_conv(x, w[p + "canon2"])
            f = experts(hin, w, p + "mlp.", lc["mlp"])
            x = group_norm(alpha * x + w[p + "ls2"] * f, w[p + "norm2"], groups, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    if n_layers is not None:
        return x
    return group_norm(x, w["final.norm"], groups, eps) @ w["head"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """greedy continuation, every step recomputed from all tokens (lowest index wins ties)"""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, w, toks, torch.float64)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
