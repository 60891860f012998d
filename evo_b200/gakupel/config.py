"""Configuration of a Gakupel model: read from the checkpoint folder's config.json (keys as the checkpoints carry them).

Every size and constant comes from here or from a tensor's shape; nothing is specialised to one checkpoint.  A layer's mixer is one of
  "attention"  causal softmax attention, per-head query / key norms, partly rotated, values = the raw key projections
  "delta"      gated delta rule behind short convolutions
  "parallel"   attention with whole-row norms, a query temperature, a distance bias and a sink, beside a matrix memory (mLSTM)
and its feed-forward is dense, a mixture of experts, or absent.  `runs` is the execution order (one run per layer); caches and states
are keyed by run."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

from ..nelovik.config import DeltaConfig, Run


@dataclass
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int = 0              # leading entries of a head that are rotated (0: none)
    rot_base: float = 10000.0
    q_temp_coef: float = 0.0       # query temperature 1 + coef * ln(floor((pos + 1) / every) + 1); every == 0: none
    q_temp_every: int = 0


@dataclass
class MemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float                # soft cap of the gate pre-activations (0: none)


@dataclass
class MlpConfig:
    kind: str                      # "dense" | "moe"
    ff: int = 0                    # dense: hidden size; moe: hidden size of one expert
    experts: int = 0
    top: int = 0
    router_scale: float = 1.0
    groups: int = 0                # runs of neighbouring experts (0 or 1: the choice is not limited)
    keep: int = 0                  # runs whose experts can be chosen
    shared_ff: int = 0             # hidden size of the always-on expert (0: none)


@dataclass
class LayerConfig:
    kind: str                      # "attention" | "delta" | "parallel"
    attention: Optional[AttentionConfig] = None        # "attention", and the left side of "parallel"
    delta: Optional[DeltaConfig] = None
    memory: Optional[MemoryConfig] = None               # the right side of "parallel"
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: Optional[MlpConfig] = None


def _attention(a: dict) -> AttentionConfig:
    rot, qt = a.get("rot") or {}, a.get("q_temp") or {}
    heads, dim = int(a["heads"]), int(a["dim"])
    c = AttentionConfig(heads, int(a.get("kv_heads", heads)), dim, int(a.get("vdim", dim)), float(a.get("scale", dim ** -0.5)),
                        int(rot.get("dims", 0) or 0), float(rot.get("base", 10000.0)), float(qt.get("coef", 0.0)), int(qt.get("every", 0) or 0))
    if c.heads % c.kv_heads:
        raise ValueError(f"{c.heads} query heads do not split over {c.kv_heads} key/value heads")
    if c.rot_dims % 2 or c.rot_dims > c.dim:
        raise ValueError(f"rot.dims ({c.rot_dims}) must be even and at most dim ({c.dim})")
    return c


def _mlp(mlp: Optional[dict]) -> Optional[MlpConfig]:
    if mlp is None:
        return None
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return MlpConfig("dense", ff=int(mlp["ff"]))
    if kind != "moe":
        raise NotImplementedError(f"feed-forward kind {kind!r}")
    r, sh = mlp["router"], mlp.get("shared")
    g = r.get("groups") or {}
    f = MlpConfig("moe", ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]), router_scale=float(r.get("scale", 1.0)),
                  groups=int(g.get("count", 0) or 0), keep=int(g.get("keep", 0) or 0), shared_ff=int(sh["ff"]) if sh else 0)
    if not 0 < f.top <= f.experts:
        raise ValueError(f"router picks {f.top} of {f.experts} experts")
    if f.groups > 1:
        if f.experts % f.groups or not 0 < f.keep <= f.groups or f.keep * (f.experts // f.groups) < f.top:
            raise ValueError(f"{f.experts} experts in {f.groups} groups of which {f.keep} stay cannot give {f.top} choices")
    return f


@dataclass
class GakupelConfig:
    vocab_size: int
    width: int
    layers: List[LayerConfig]
    eps: float
    max_seqlen: int = 8192
    max_batch_size: int = 1
    runs: List[Run] = field(default_factory=list)

    def __post_init__(self):
        self.runs = [Run(i) for i in range(len(self.layers))]

    def get(self, key, default=None):
        return getattr(self, key, default)

    @classmethod
    def from_dict(cls, d: dict) -> "GakupelConfig":
        layers = []
        for entry in d["layers"]:
            kind, m = entry["type"], entry["mixer"]
            mlp = _mlp(entry.get("mlp"))
            if kind == "attention":
                a = _attention(m)
                if a.vdim != a.dim:
                    raise ValueError(f"values are the key projections: vdim ({a.vdim}) must equal dim ({a.dim})")
                layers.append(LayerConfig(kind, attention=a, mlp=mlp))
            elif kind == "delta":
                heads = int(m["heads"])
                kv = int(m.get("kv_heads", heads))
                if heads % kv:
                    raise ValueError(f"{heads} heads do not split over {kv} query/key heads")
                layers.append(LayerConfig(kind, delta=DeltaConfig(heads, kv, int(m["dim"]), int(m["vdim"]), int(m["conv"])), mlp=mlp))
            elif kind == "parallel":
                s = m["right"]
                mem = MemoryConfig(int(s["heads"]), int(s["dim"]), int(s["vdim"]), float(s.get("gate_cap", 0.0) or 0.0))
                layers.append(LayerConfig(kind, attention=_attention(m["left"]), memory=mem, left_scale=float(m.get("left_scale", 1.0)),
                                          right_scale=float(m.get("right_scale", 1.0)), mlp=mlp))
            else:
                raise NotImplementedError(f"mixer type {kind!r}")
        return cls(vocab_size=int(d["vocab"]), width=int(d["width"]), layers=layers, eps=float(d["norm"]["eps"]), max_seqlen=int(d.get("max_seqlen", 8192)))

    @classmethod
    def from_dir(cls, model_dir: str) -> "GakupelConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    @property
    def unused_tensor_names(self):
        """Tensors a checkpoint may carry although this configuration never reads them (the second norm of a layer without feed-forward)."""
        out = []
        for i, layer in enumerate(self.layers):
            if layer.mlp is None:
                out += [f"l{i}.norm2", f"l{i}.norm2.b"]
        return tuple(out)

    def tensor_shapes(self) -> dict:
        """checkpoint tensor name -> shape, in checkpoint naming."""
        d, out = self.width, {"embed": (self.vocab_size, self.width)}
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            out.update({p + "norm1": (d,), p + "norm1.b": (d,)})
            if layer.mlp is not None:
                out.update({p + "norm2": (d,), p + "norm2.b": (d,)})
            q = p + "mix."
            if layer.kind == "attention":
                a = layer.attention
                out.update({q + "q": (a.heads * a.dim, d), q + "k": (a.kv_heads * a.dim, d), q + "q.norm": (a.dim,), q + "k.norm": (a.dim,),
                            q + "o": (d, a.heads * a.vdim)})
            elif layer.kind == "delta":
                m = layer.delta
                qk, vw = m.kv_heads * m.dim, m.heads * m.vdim
                out.update({q + "q": (qk, d), q + "q.conv": (qk, m.taps), q + "k": (qk, d), q + "k.conv": (qk, m.taps),
                            q + "v": (vw, d), q + "v.conv": (vw, m.taps), q + "b": (m.heads, d), q + "a": (m.heads, d),
                            q + "A_log": (m.heads,), q + "dt_bias": (m.heads,), q + "norm": (m.vdim,), q + "g": (vw, d), q + "o": (d, vw)})
            else:
                a, s = layer.attention, layer.memory
                l, r = q + "left.", q + "right."
                out.update({l + "q": (a.heads * a.dim, d), l + "k": (a.kv_heads * a.dim, d), l + "v": (a.kv_heads * a.vdim, d),
                            l + "q.norm": (a.heads * a.dim,), l + "k.norm": (a.kv_heads * a.dim,), l + "r1": (a.heads,), l + "r2": (a.heads,),
                            l + "o": (d, a.heads * a.vdim)})
                out.update({r + "q": (s.heads * s.dim, d), r + "k": (s.heads * s.dim, d), r + "v": (s.heads * s.vdim, d), r + "g": (s.heads * s.vdim, d),
                            r + "o": (d, s.heads * s.vdim), r + "norm": (s.heads * s.vdim,), r + "i": (s.heads, d), r + "i.b": (s.heads,),
                            r + "f": (s.heads, d), r + "f.b": (s.heads,)})
            f = layer.mlp
            if f is not None and f.kind == "dense":
                out.update({p + "mlp.up": (f.ff, d), p + "mlp.down": (d, f.ff)})
            elif f is not None:
                for e in range(f.experts):
                    out.update({f"{p}mlp.e{e}.gate": (f.ff, d), f"{p}mlp.e{e}.up": (f.ff, d), f"{p}mlp.e{e}.down": (d, f.ff)})
                out.update({p + "mlp.router": (f.experts, d), p + "mlp.correction": (f.experts,)})
                if f.shared_ff:
                    out.update({p + "mlp.shared.gate": (f.shared_ff, d), p + "mlp.shared.up": (f.shared_ff, d), p + "mlp.shared.down": (d, f.shared_ff),
                                p + "mlp.shared.sg": (1, d)})
            out[p + "dwa"] = (i + 2,)
        out["final.norm"] = (d,)
        out["final.norm.b"] = (d,)
        out["head"] = (self.vocab_size, d)
        return out
