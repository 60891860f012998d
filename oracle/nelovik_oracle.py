"""Plain, slow statement of the Nelovik design in PyTorch, one function per mechanism, whole sequences only, float64 by
default.  It shares no code with evo_b200: the product is compared against it.

Notation: T tokens, D width, H heads, G key/value heads (or groups), dk / dv per-head key / value sizes, N state size.
  rms(u)         = u / sqrt(mean(u^2) + eps)                                    (over the last axis)
  unit(u)        = u / sqrt(sum(u^2) + 1e-6)
  conv(x, c)     : y_t = sum_j c[:, j] * x_{t - (taps-1) + j}  (+ bias), zeros before the first token
  xielu(z; p, q) = softplus(p) z^2 + z/2  (z > 0);  (1/2 + softplus(q)) (e^z - 1 - z) + z/2  (z <= 0)
  layer          : x <- x + mixer(rms(x) w1) + ff(rms(x) w2)       (both branches read the same x)
  gated delta    : S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
  ssd            : S <- exp(-exp(A) dt) S + dt B x^T;  y = S^T C + D x
  pooled window  : query i sees tokens j with 0 <= i - j < W and the means of the blocks [bP, bP + P) with bP + P - 1 <= i - W;
                   scores are scaled, soft-capped, and share one softmax whose denominator also holds exp(sink_h)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def rms(u: torch.Tensor, eps: float) -> torch.Tensor:
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def unit(u: torch.Tensor) -> torch.Tensor:
    return u / torch.sqrt((u * u).sum(-1, keepdim=True) + 1e-6)


def silu(z):
    return z * torch.sigmoid(z)


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    pos = F.softplus(p) * z * z + 0.5 * z
    neg = (0.5 + F.softplus(q)) * (torch.expm1(z) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def short_conv(x: torch.Tensor, c: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x (T, C), c (C, taps): the last column of c multiplies the current token."""
    T, taps = x.shape[0], c.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += c[:, j] * x[s]
    if bias is not None:
        out = out + bias
    return out


def rotate_half(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x (T, H, d): the first `dims` entries of each head are rotated, entry i paired with entry i + dims/2."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = pos.to(x.dtype)[:, None] * f[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def gated_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h (T, D) -> (T, D).  w: the mixer's tensors without the layer prefix ('q', 'q.conv', ...)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, dk)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, dk)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w["b"].T)                                          # (T, H)
    g = torch.exp(-torch.exp(w["A_log"]) * F.softplus(h @ w["a"].T + w["dt_bias"]))
    gate = silu(h @ w["g"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, hd] = S.T @ q[t, kv]
    out = rms(out, eps) * w["norm"] * gate
    return out.reshape(T, H * dv) @ w["o"].T


def ssd(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dv, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * dv
    zxbcdt = h @ w["in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].view(T, H, dv)
    Bm = xbc[:, inner:inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + w["dt_bias"])                                          # (T, H)
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)
    y = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        gr = hd // (H // G)
        S = torch.zeros(N, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(Bm[t, gr], x[t, hd])
            y[t, hd] = S.T @ Cm[t, gr] + w["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.view(T, NG, inner // NG), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def visible_tokens(i: int, window: int) -> List[int]:
    return [j for j in range(max(0, i - window + 1), i + 1)]


def visible_blocks(i: int, window: int, pool: int) -> List[int]:
    if pool <= 0:
        return []
    return [b for b in range(0, i // pool + 1) if b * pool + pool - 1 <= i - window]


def pooled_window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, rows=None) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window, pool = int(m["mask"]["size"]), int(m["mask"].get("pool", 0))
    q = h @ w["q"].T + w["q.b"]
    k = h @ w["k"].T + w["k.b"]
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    q = (rms(q, eps) * w["q.norm"]).view(T, H, dk)
    k = (rms(k, eps) * w["k.norm"]).view(T, G, dk)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, pos, int(rot["dims"]), float(rot["base"]))
        k = rotate_half(k, pos, int(rot["dims"]), float(rot["base"]))
    cap = float(m.get("softcap", 0.0) or 0.0)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        for i in (range(T) if rows is None else rows):
            js, bs = visible_tokens(i, window), visible_blocks(i, window, pool)
            keys = [k[j, g] for j in js] + [k[b * pool:(b + 1) * pool, g].mean(0) for b in bs]
            vals = [v[j, g] for j in js] + [v[b * pool:(b + 1) * pool, g].mean(0) for b in bs]
            s = torch.stack(keys) @ q[i, hd] * m["scale"]
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            mx = torch.maximum(s.max(), w["sink"][hd])
            e = torch.exp(s - mx)
            den = e.sum() + torch.exp(w["sink"][hd] - mx)
            out[i, hd] = (e[:, None] * torch.stack(vals)).sum(0) / den
    return out.reshape(T, H * dv) @ w["o"].T


def parallel_mixer(h, w, m, eps, rows=None):
    left = {k[len("left."):]: t for k, t in w.items() if k.startswith("left.")}
    right = {k[len("right."):]: t for k, t in w.items() if k.startswith("right.")}
    a = pooled_window_attention(h, left, m["left"], eps, rows=rows)
    b = ssd(h, right, m["right"], eps)
    return 0.5 * (rms(a, eps) * w["left.out"] + rms(b, eps) * w["right.out"])


def feed_forward(h, w):
    return xielu(h @ w["up"].T, w["act"][0], w["act"][1]) @ w["down"].T


def is_delta(kind: str) -> bool:
    return kind == "delta" or (kind.startswith("delta_") and kind[len("delta_"):].isdigit())


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, taps: Optional[list] = None) -> torch.Tensor:
    """tokens (T,) -> logits (T, V); `taps` (a list) receives the residual stream after every layer."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mix = {k[len(p + "mix."):]: t for k, t in W.items() if k.startswith(p + "mix.")}
        h1 = rms(x, eps) * W[p + "norm1"]
        kind = layer["type"]
        if is_delta(kind):
            y = gated_delta(h1, mix, layer["mixer"], eps)
        elif kind == "parallel":
            y = parallel_mixer(h1, mix, layer["mixer"], eps)
        else:
            raise NotImplementedError(kind)
        if layer.get("mlp") is not None:
            h2 = rms(x, eps) * W[p + "norm2"]
            y = y + feed_forward(h2, {k[len(p + "mlp."):]: t for k, t in W.items() if k.startswith(p + "mlp.")})
        x = x + y
        if taps is not None:
            taps.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T
