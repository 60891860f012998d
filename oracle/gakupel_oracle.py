"""Plain, slow statement of the Gakupel design in PyTorch, one function per mechanism, whole sequences only, float64 by
default.  It shares no code with evo_b200: the product is compared against it.

Notation: T tokens, D width, H heads, G key/value heads, dk / dv per-head key / value sizes, positions 0 .. T-1.
  ln(u; w, b)    = (u - mean u) / sqrt(var u + eps) * w + b                     (biased variance, over the last axis)
  rms(u)         = u / sqrt(mean(u^2) + eps)
  unit(u)        = u / sqrt(sum(u^2) + 1e-6)
  layer i        : y = x + ln1(mixer(x));  X_{i+1} = y + ln2(ff(y));  x <- sum_{j <= i+1} a_i[j] X_j       (X_0: embedding rows)
  attention      : q, k normed per head and partly rotated; values are the un-normed, un-rotated key projections; causal softmax
  biased sink    : whole-row q / k norms, q_t *= 1 + c ln(floor((t+1)/n) + 1), s_ij = scale q_i.k_j - r1 ln(1 + r2 (i-j)),
                   p_ij = e^{s_ij} / (1 + sum_j e^{s_ij})
  matrix memory  : m_t = max(f_t + m_{t-1}, i_t);  S_t = e^{f_t + m_{t-1} - m_t} S_{t-1} + e^{i_t - m_t} k_t v_t^T (n_t alike with k_t);
                   o_t = S_t^T q_t / (max(|n_t.q_t|, e^{-m_t}) + 1e-6),  m_0 = 0,  gates soft-capped: c tanh(z / c)
  gated delta    : S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
  router         : s = sigmoid(W h); c = s + correction; groups ranked by the sum of their two largest c; top-k of c inside the
                   kept groups; weights s / (sum of chosen s + 1e-20) * scale
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def layer_norm(u, w, b, eps):
    mu = u.mean(-1, keepdim=True)
    var = ((u - mu) ** 2).mean(-1, keepdim=True)
    return (u - mu) / torch.sqrt(var + eps) * w + b


def rms(u, eps):
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def unit(u):
    return u / torch.sqrt((u * u).sum(-1, keepdim=True) + 1e-6)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def short_conv(x, c):
    """x (T, C), c (C, taps): the last column of c multiplies the current token; zeros before the first token."""
    T, taps = x.shape[0], c.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += c[:, j] * x[s]
    return out


def rotate_half(x, pos, dims, base):
    """x (T, H, d): the first `dims` entries of each head are turned, entry i paired with entry i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = pos.to(x.dtype)[:, None] * f[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def attention(h, w, m, eps):
    """Causal softmax attention whose values are the raw key projections.  h (T, D) -> (T, D)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    assert dv == dk, "the values are the key projections"
    rot = m.get("rot") or {}
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, dk)
    kraw = (h @ w["k"].T).view(T, G, dk)
    v = kraw
    q = rotate_half(rms(q, eps) * w["q.norm"], pos, int(rot.get("dims", 0)), float(rot.get("base", 10000.0)))
    k = rotate_half(rms(kraw, eps) * w["k.norm"], pos, int(rot.get("dims", 0)), float(rot.get("base", 10000.0)))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, hd]) * m["scale"]
            p = torch.softmax(s, 0)
            out[i, hd] = p @ v[:i + 1, g]
    return out.reshape(T, H * dv) @ w["o"].T


def biased_sink_attention(h, w, m, eps):
    """The attention side of a parallel mixer.  h (T, D) -> (T, D)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    qt = m.get("q_temp") or {}
    q = rms(h @ w["q"].T, eps) * w["q.norm"]
    k = rms(h @ w["k"].T, eps) * w["k.norm"]
    v = (h @ w["v"].T).view(T, G, dv)
    if qt:
        pos = torch.arange(T, dtype=torch.int64)
        steps = torch.div(pos + 1, int(qt["every"]), rounding_mode="floor").to(h.dtype)
        q = q * (1.0 + float(qt["coef"]) * torch.log(steps + 1.0))[:, None]
    q, k = q.view(T, H, dk), k.view(T, G, dk)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        r1, r2 = w["r1"][hd], w["r2"][hd]
        for i in range(T):
            dist = (i - torch.arange(i + 1)).to(h.dtype)
            s = (k[:i + 1, g] @ q[i, hd]) * m["scale"] - r1 * torch.log(1.0 + r2 * dist)
            e = torch.exp(s)
            out[i, hd] = (e / (1.0 + e.sum())) @ v[:i + 1, g]
    return out.reshape(T, H * dv) @ w["o"].T


def matrix_memory(h, w, m, eps):
    """The recurrent side of a parallel mixer.  h (T, D) -> (T, D)."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w["q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).view(T, H, dk)
    v = (h @ w["v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                       # (T, H) log input gate
    fg = F.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))        # (T, H) log forget gate
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        n = torch.zeros(dk, dtype=h.dtype)
        mrun = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            mnew = torch.maximum(fg[t, hd] + mrun, ig[t, hd])
            a, b = torch.exp(fg[t, hd] + mrun - mnew), torch.exp(ig[t, hd] - mnew)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mrun = mnew
            den = torch.maximum((n @ q[t, hd]).abs(), torch.exp(-mrun)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    o = rms(out, eps).reshape(T, H * dv) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def parallel_mixer(h, w, m, eps):
    left = biased_sink_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps)
    right = matrix_memory(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def gated_delta(h, w, m, eps):
    """h (T, D) -> (T, D)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, dk)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, dk)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w["b"].T)
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
    o = rms(out, eps) * w["norm"] * gate
    return o.reshape(T, H * dv) @ w["o"].T


def dense_ff(h, w):
    return gelu_erf(h @ w["up"].T) @ w["down"].T


def route(h, w, r):
    """h (T, D) -> (T, experts) weights, zero for experts that are not chosen."""
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {}
    s = torch.sigmoid(h @ w["router"].T)
    c = s + w["correction"]
    if groups and int(groups["count"]) > 1:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        cg = c.view(-1, n, per)
        rank = cg.topk(min(2, per), -1).values.sum(-1)                          # (T, n)
        kept = torch.zeros_like(rank, dtype=torch.bool)
        kept.scatter_(1, rank.topk(keep, -1).indices, True)
        c = torch.where(kept[:, :, None].expand(-1, -1, per).reshape(-1, E), c, torch.full_like(c, -math.inf))
    idx = c.topk(top, -1).indices
    picked = s.gather(1, idx)
    wts = picked / (picked.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    out = torch.zeros_like(s)
    out.scatter_(1, idx, wts)
    return out


def glu_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def moe_ff(h, w, f):
    wts = route(h, w, f["router"])
    out = torch.zeros_like(h)
    for e in range(int(f["router"]["experts"])):
        out = out + wts[:, e:e + 1] * glu_expert(h, w, f"e{e}.")
    if f.get("shared"):
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * glu_expert(h, w, "shared.")
    return out


MIXERS = {"attention": attention, "delta": gated_delta, "parallel": parallel_mixer}


def forward(tokens: List[int], W: Dict[str, torch.Tensor], cfg: dict, dtype=torch.float64, taps: Optional[list] = None):
    """Logits (T, V) of a whole sequence.  taps: receives every layer's result X_{i+1} (before the depth average)."""
    W = {k: v.to(dtype) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(tokens)]
    results = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        sub = lambda pre: {k[len(pre):]: v for k, v in W.items() if k.startswith(pre)}
        y = MIXERS[layer["type"]](x, sub(p + "mix."), layer["mixer"], eps)
        x = x + layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps)
        f = layer.get("mlp")
        if f is not None:
            y = dense_ff(x, sub(p + "mlp.")) if f.get("kind", "dense") == "dense" else moe_ff(x, sub(p + "mlp."), f)
            x = x + layer_norm(y, W[p + "norm2"], W[p + "norm2.b"], eps)
        results.append(x)
        if taps is not None:
            taps.append(x)
        a = W[p + "dwa"]
        x = sum(a[j] * results[j] for j in range(len(results)))
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return x @ W["head"].T


def random_weights(cfg: dict, shapes: Dict[str, tuple], seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16-representable weights of a usable scale for the tensor table `shapes` (name -> shape)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes.items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm" or name.endswith((".q.norm", ".k.norm", "mix.norm", "right.norm")):
            v = 1.0 + torch.randn(shape, generator=g) * 0.1
        elif leaf == "b" and len(shape) == 1:
            v = torch.randn(shape, generator=g) * 0.2
        elif leaf == "A_log":
            v = torch.log(0.5 + 3.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            v = torch.randn(shape, generator=g) * 0.5 - 1.0
        elif leaf == "conv":
            v = torch.randn(shape, generator=g) * 0.4
        elif leaf == "r1":
            v = 0.2 + torch.rand(shape, generator=g)
        elif leaf == "r2":
            v = 0.05 + 0.5 * torch.rand(shape, generator=g)
        elif leaf == "correction":
            v = torch.randn(shape, generator=g) * 0.3
        elif leaf == "dwa":
            v = torch.randn(shape, generator=g) * 0.2
            v[-1] += 1.0
        elif leaf in ("i", "f") and name.endswith(("right.i", "right.f")):
            v = torch.randn(shape, generator=g) * 2.0 / math.sqrt(shape[-1])
        elif name == "embed":
            v = torch.randn(shape, generator=g)
        else:
            v = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = v.to(torch.bfloat16).to(torch.float32)
    return out
