"""Configuration of a Nelovik model: read from the checkpoint folder's config.json (keys as the checkpoints carry them).

Every size comes from here or from a tensor's shape; nothing is specialised to one checkpoint.  A layer is one of
  "delta"      gated delta rule
  "parallel"   pooled-window attention beside a state-space mixer
(a numbered name such as "delta_2" is the same mechanism with sizes of its own)
and may or may not have a feed-forward.  `runs` is the execution order (one run per layer); caches and states are keyed by run."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int                       # per-head query/key size
    vdim: int                      # per-head value size
    taps: int                      # short-convolution taps


@dataclass
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                 # 0: none
    window: int                    # visible distance
    pool: int                      # tokens per pooled block before the window (0: none)
    rot_dims: int                  # leading entries of a head that are rotated (0: none)
    rot_base: float


@dataclass
class SsdConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    taps: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass
class LayerConfig:
    kind: str                      # "delta" | "parallel"
    delta: Optional[DeltaConfig] = None
    left: Optional[AttentionConfig] = None
    right: Optional[SsdConfig] = None
    ff: Optional[int] = None       # feed-forward width, None: no feed-forward


@dataclass
class Run:
    layer: int


def _base_kind(kind: str) -> str:
    """"delta_2" -> "delta": a numbered name is the same mechanism with sizes of its own."""
    head, _, tail = kind.rpartition("_")
    return head if head and tail.isdigit() else kind


@dataclass
class NelovikConfig:
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
    def from_dict(cls, d: dict) -> "NelovikConfig":
        layers = []
        for entry in d["layers"]:
            kind, m = entry["type"], entry["mixer"]
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            ff = None if mlp is None else int(mlp["ff"])
            if _base_kind(kind) == "delta":
                heads = int(m["heads"])
                layers.append(LayerConfig("delta", delta=DeltaConfig(heads, int(m.get("kv_heads", heads)), int(m["dim"]), int(m["vdim"]), int(m["conv"])), ff=ff))
            elif _base_kind(kind) == "parallel":
                a, s = m["left"], m["right"]
                mask, rot = a.get("mask") or {}, a.get("rot") or {}
                heads = int(a["heads"])
                left = AttentionConfig(heads, int(a.get("kv_heads", heads)), int(a["dim"]), int(a["vdim"]), float(a.get("scale", int(a["dim"]) ** -0.5)),
                                       float(a.get("softcap", 0.0) or 0.0), int(mask.get("size", 0)), int(mask.get("pool", 0) or 0),
                                       int(rot.get("dims", 0) or 0), float(rot.get("base", 10000.0)))
                if left.pool > 0 and left.window <= 0:
                    raise ValueError("pooled blocks need a window")
                right = SsdConfig(int(s["heads"]), int(s["vdim"]), int(s["state"]), int(s.get("groups", 1)), int(s.get("norm_groups", 1)), int(s["conv"]))
                layers.append(LayerConfig("parallel", left=left, right=right, ff=ff))
            else:
                raise NotImplementedError(f"mixer type {kind!r}")
        return cls(vocab_size=int(d["vocab"]), width=int(d["width"]), layers=layers, eps=float(d["norm"]["eps"]), max_seqlen=int(d.get("max_seqlen", 8192)))

    @classmethod
    def from_dir(cls, model_dir: str) -> "NelovikConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def tensor_shapes(self) -> dict:
        """checkpoint tensor name -> shape, in checkpoint naming."""
        d, out = self.width, {"embed": (self.vocab_size, self.width)}
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            out[p + "norm1"] = (d,)
            if layer.ff is not None:
                out[p + "norm2"] = (d,)
            if layer.kind == "delta":
                m = layer.delta
                qk, vw = m.kv_heads * m.dim, m.heads * m.vdim
                out.update({p + "mix.q": (qk, d), p + "mix.q.conv": (qk, m.taps), p + "mix.k": (qk, d), p + "mix.k.conv": (qk, m.taps),
                            p + "mix.v": (vw, d), p + "mix.v.conv": (vw, m.taps), p + "mix.b": (m.heads, d), p + "mix.a": (m.heads, d),
                            p + "mix.A_log": (m.heads,), p + "mix.dt_bias": (m.heads,), p + "mix.norm": (m.vdim,),
                            p + "mix.g": (vw, d), p + "mix.o": (d, vw)})
            else:
                a, s = layer.left, layer.right
                q = p + "mix.left."
                out.update({q + "q": (a.heads * a.dim, d), q + "q.b": (a.heads * a.dim,), q + "k": (a.kv_heads * a.dim, d), q + "k.b": (a.kv_heads * a.dim,),
                            q + "v": (a.kv_heads * a.vdim, d), q + "v.b": (a.kv_heads * a.vdim,), q + "q.norm": (a.heads * a.dim,),
                            q + "k.norm": (a.kv_heads * a.dim,), q + "sink": (a.heads,), q + "o": (d, a.heads * a.vdim), q + "out": (d,)})
                r = p + "mix.right."
                out.update({r + "in": (2 * s.inner + 2 * s.groups * s.state + s.heads, d), r + "conv": (s.conv_channels, s.taps),
                            r + "conv.b": (s.conv_channels,), r + "dt_bias": (s.heads,), r + "A_log": (s.heads,), r + "D": (s.heads,),
                            r + "norm": (s.inner,), r + "o": (d, s.inner), r + "out": (d,)})
            if layer.ff is not None:
                out.update({p + "mlp.up": (layer.ff, d), p + "mlp.down": (d, layer.ff), p + "mlp.act": (2,)})
        out["final.norm"] = (d,)
        out["head"] = (self.vocab_size, d)
        return out
