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


def base_kind(kind: str) -> str:
    head, _, tail = kind.rpartition("_")
    return head if head and tail.isdigit() else kind


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
        if base_kind(kind) == "delta":
            y = gated_delta(h1, mix, layer["mixer"], eps)
        elif base_kind(kind) == "parallel":
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


# ---- small configurations and random weights for the tests --------------------------------------------------------------
def make_config(width=48, vocab=61, layers=("parallel", "delta", "delta_2"), ff=40, no_ff_layers=(), eps=1e-5,
                heads=2, kv_heads=1, dim=8, vdim=12, taps=3,                                    # gated delta rule
                att_heads=4, att_kv_heads=2, att_dim=12, att_vdim=10, window=9, pool=3, rot_dims=8, rot_base=100.0, scale=0.3, softcap=5.0,
                ssd_heads=4, ssd_vdim=6, state=5, groups=2, norm_groups=3, ssd_taps=2) -> dict:
    """A config.json dict; entries of `layers` may also be complete layer dicts (layers with sizes of their own)."""
    out = []
    for i, kind in enumerate(layers):
        if isinstance(kind, dict):
            out.append(kind)
            continue
        if base_kind(kind) == "parallel":
            left = {"heads": att_heads, "kv_heads": att_kv_heads, "dim": att_dim, "vdim": att_vdim, "mask": {"size": window, "pool": pool},
                    "scale": scale, "softcap": softcap}
            if rot_dims:
                left["rot"] = {"dims": rot_dims, "base": rot_base}
            mixer = {"left": left, "right": {"heads": ssd_heads, "vdim": ssd_vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": ssd_taps}}
        else:
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}
        out.append({"type": kind, "mixer": mixer, "mlp": None if i in no_ff_layers else {"kind": "dense", "ff": ff}})
    return {"architecture": "Nelovik", "vocab": vocab, "width": width, "layers": out, "norm": {"eps": eps}}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    d = config["width"]
    out = {"embed": (config["vocab"], d)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (d,)
        if base_kind(layer["type"]) == "parallel":
            a, s = m["left"], m["right"]
            q = p + "mix.left."
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for name, shape in (("q", (H * dk, d)), ("q.b", (H * dk,)), ("k", (G * dk, d)), ("k.b", (G * dk,)), ("v", (G * dv, d)), ("v.b", (G * dv,)),
                                ("q.norm", (H * dk,)), ("k.norm", (G * dk,)), ("sink", (H,)), ("o", (d, H * dv)), ("out", (d,))):
                out[q + name] = shape
            r = p + "mix.right."
            inner, gn = s["heads"] * s["vdim"], s["groups"] * s["state"]
            for name, shape in (("in", (2 * inner + 2 * gn + s["heads"], d)), ("conv", (inner + 2 * gn, s["conv"])), ("conv.b", (inner + 2 * gn,)),
                                ("dt_bias", (s["heads"],)), ("A_log", (s["heads"],)), ("D", (s["heads"],)), ("norm", (inner,)), ("o", (d, inner)), ("out", (d,))):
                out[r + name] = shape
        else:
            H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, shape in (("q", (G * dk, d)), ("q.conv", (G * dk, taps)), ("k", (G * dk, d)), ("k.conv", (G * dk, taps)), ("v", (H * dv, d)),
                                ("v.conv", (H * dv, taps)), ("b", (H, d)), ("a", (H, d)), ("A_log", (H,)), ("dt_bias", (H,)), ("norm", (dv,)),
                                ("g", (H * dv, d)), ("o", (d, H * dv))):
                out[p + "mix." + name] = shape
        if layer.get("mlp") is not None:
            out[p + "norm2"] = (d,)
            out.update({p + "mlp.up": (layer["mlp"]["ff"], d), p + "mlp.down": (d, layer["mlp"]["ff"]), p + "mlp.act": (2,)})
    out["final.norm"] = (d,)
    out["head"] = (config["vocab"], d)
    return out


def random_weights(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 tensors of a scale at which every mechanism matters (decays well inside (0, 1), sinks comparable to the scores)."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and leaf != "conv":
            v = torch.randn(shape, generator=g) * (1.0 if name == "embed" else 1.5 / math.sqrt(shape[1]))
        elif leaf == "conv":
            v = torch.randn(shape, generator=g) * 0.5
        elif leaf == "A_log":
            v = torch.log(0.3 + 2.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            v = torch.randn(shape, generator=g) * 0.7 - 0.5
        elif leaf in ("sink", "D"):
            v = torch.randn(shape, generator=g)
        elif leaf == "act":
            v = torch.tensor([0.3, 0.8]) + torch.randn(2, generator=g) * 0.2
        elif leaf == "b":                               # projection biases
            v = torch.randn(shape, generator=g) * 0.3
        else:                                           # norm weights
            v = 1.0 + torch.randn(shape, generator=g) * 0.2
        W[name] = v.to(torch.bfloat16)
    return W
