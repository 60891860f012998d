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
    """Logits (T, V) of a whole sequence.  taps: receives the stream every layer hands on (after the mix of the results so far)."""
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
        a = W[p + "dwa"]
        x = sum(a[j] * results[j] for j in range(len(results)))
        if taps is not None:
            taps.append(x)
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return x @ W["head"].T


def make_config(layers=("parallel", "attention", "delta"), mlps=("dense", "moe", "moe"), width=64, vocab=97, ff=96, eps=1e-5,
                att_heads=4, att_kv_heads=2, att_dim=16, rot_dims=8, rot_base=1000.0, att_scale=0.3,
                left_heads=4, left_kv_heads=2, left_dim=16, left_vdim=12, left_scale_qk=0.25, temp_coef=0.4, temp_every=8, left_scale=1.3, right_scale=0.6,
                mem_heads=2, mem_dim=12, mem_vdim=20, gate_cap=6.0,
                heads=4, kv_heads=2, dim=8, vdim=16, taps=3,
                experts=8, top=3, groups=4, keep=2, router_scale=1.5, expert_ff=24, shared_ff=40) -> dict:
    """A small configuration in the checkpoints' own keys; every layer of a kind gets the same sizes (tests change single entries)."""
    out = []
    for kind, mlp in zip(layers, mlps):
        if kind == "attention":
            m = {"heads": att_heads, "kv_heads": att_kv_heads, "dim": att_dim, "vdim": att_dim, "scale": att_scale}
            if rot_dims:
                m["rot"] = {"base": rot_base, "dims": rot_dims}
        elif kind == "delta":
            m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}
        else:
            left = {"heads": left_heads, "kv_heads": left_kv_heads, "dim": left_dim, "vdim": left_vdim, "scale": left_scale_qk}
            if temp_every:
                left["q_temp"] = {"coef": temp_coef, "every": temp_every}
            m = {"left": left, "left_scale": left_scale, "right": {"heads": mem_heads, "dim": mem_dim, "vdim": mem_vdim, "gate_cap": gate_cap}, "right_scale": right_scale}
        if mlp == "dense":
            f = {"kind": "dense", "ff": ff}
        elif mlp == "moe":
            router = {"experts": experts, "top": top, "scale": router_scale}
            if groups:
                router["groups"] = {"count": groups, "keep": keep}
            f = {"kind": "moe", "expert": {"ff": expert_ff}, "router": router}
            if shared_ff:
                f["shared"] = {"ff": shared_ff}
        else:
            f = None
        out.append({"type": kind, "mixer": m, "mlp": f})
    return {"architecture": "Gakupel", "layers": out, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Checkpoint tensor name -> shape for a configuration."""
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1.b"] = (d,)
        q = p + "mix."
        if layer["type"] == "attention":
            H, G, dk = m["heads"], m["kv_heads"], m["dim"]
            out.update({q + "q": (H * dk, d), q + "k": (G * dk, d), q + "q.norm": (dk,), q + "k.norm": (dk,), q + "o": (d, H * dk)})
        elif layer["type"] == "delta":
            H, G, dk, dv, t = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({q + "q": (G * dk, d), q + "q.conv": (G * dk, t), q + "k": (G * dk, d), q + "k.conv": (G * dk, t), q + "v": (H * dv, d), q + "v.conv": (H * dv, t),
                        q + "b": (H, d), q + "a": (H, d), q + "A_log": (H,), q + "dt_bias": (H,), q + "norm": (dv,), q + "g": (H * dv, d), q + "o": (d, H * dv)})
        else:
            a, s = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            out.update({q + "left.q": (H * dk, d), q + "left.k": (G * dk, d), q + "left.v": (G * dv, d), q + "left.q.norm": (H * dk,), q + "left.k.norm": (G * dk,),
                        q + "left.r1": (H,), q + "left.r2": (H,), q + "left.o": (d, H * dv)})
            H, dk, dv = s["heads"], s["dim"], s["vdim"]
            out.update({q + "right.q": (H * dk, d), q + "right.k": (H * dk, d), q + "right.v": (H * dv, d), q + "right.g": (H * dv, d), q + "right.o": (d, H * dv),
                        q + "right.norm": (H * dv,), q + "right.i": (H, d), q + "right.i.b": (H,), q + "right.f": (H, d), q + "right.f.b": (H,)})
        f = layer.get("mlp")
        if f is not None:
            out[p + "norm2"] = out[p + "norm2.b"] = (d,)
            if f.get("kind", "dense") == "dense":
                out.update({p + "mlp.up": (f["ff"], d), p + "mlp.down": (d, f["ff"])})
            else:
                e = f["expert"]["ff"]
                for k in range(f["router"]["experts"]):
                    out.update({f"{p}mlp.e{k}.gate": (e, d), f"{p}mlp.e{k}.up": (e, d), f"{p}mlp.e{k}.down": (d, e)})
                out.update({p + "mlp.router": (f["router"]["experts"], d), p + "mlp.correction": (f["router"]["experts"],)})
                if f.get("shared"):
                    e = f["shared"]["ff"]
                    out.update({p + "mlp.shared.gate": (e, d), p + "mlp.shared.up": (e, d), p + "mlp.shared.down": (d, e), p + "mlp.shared.sg": (1, d)})
        out[p + "dwa"] = (i + 2,)
    out["final.norm"] = out["final.norm.b"] = (d,)
    out["head"] = (V, d)
    return out


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16-representable weights of a usable scale."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
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
        out[name] = v.to(torch.bfloat16)
    return out
