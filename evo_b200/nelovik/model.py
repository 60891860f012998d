"""Nelovik: a decoder-only model whose layers run the mixer and the feed-forward side by side on two norms of the same fp32
stream, x <- x + mixer(norm1(x)) + ff(norm2(x)), with two kinds of mixer -- the gated delta rule, and a pair of mixers run side
by side (windowed attention over tokens and pooled blocks with a softmax sink, beside a state-space-duality recurrence) whose
outputs are normed and averaged -- and an xIELU feed-forward; executed by libevo_b200.so.

It follows the object protocol of the framework's other models (see stream_model.StreamDecoder), so the same generation loop,
scheduler, trace replay and command line drive it.  State, keyed by RUN index r:
    d["mha"].key_value_memory_dict[r]        (B, max_seqlen, G*dim + G*vdim): keys (normed, rotated), then values
    d["mha"].key_value_memory_dict[-(r+1)]   (B, max_seqlen/pool + 1, same row): means of the completed blocks of `pool` rows
    d["hyena"].fir_state_dict[r]             (B, taps-1, channels) fp32: the last inputs of the short convolution
    d["hyena"].state_dict[r]                 (B, heads, dim | state, vdim) fp32: the recurrence's matrix state
The branches of a layer are summed into x by the kernel that also emits the next layer's two norms (evo_sum_norm), so x is read
and written once per layer.  Linear layers: bf16 activations -> the framework's tcgen05 GEMMs (weights zero-padded once to their
tiles); fp32 activations (dtype=torch.float32) -> evo_gemm_simt, true fp32 multiply-add.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _lib
from .._lib import QkPrepParams, SsdParams, SumNormParams, WindowAttnParams, check, ptr
from ..stream_model import StreamDecoder, _Packed, _round_up
from .config import NelovikConfig


class Nelovik(StreamDecoder):
    architecture = "Nelovik"
    gemm_env = "EVO_B200_NELOVIK_GEMM"

    def __init__(self, config: NelovikConfig, dtype: torch.dtype = torch.bfloat16):
        super().__init__(config, dtype)
        self.fir_taps = max([l.delta.taps if l.kind == "delta" else l.right.taps for l in config.layers] or [0])

    # ---- parameters ----------------------------------------------------------------------------
    def init_random(self, seed: int = 0, device=None) -> "Nelovik":
        """Random weights of a usable scale (benchmarks, tests)."""
        g = torch.Generator().manual_seed(seed)
        for name, t in self.weights.items():
            shape = t.shape
            leaf = name.split(".")[-1]
            if leaf in ("norm1", "norm2") or name == "final.norm" or name.endswith(("left.out", "right.out", "q.norm", "k.norm", "mix.norm", "right.norm")):
                v = 1.0 + torch.randn(shape, generator=g) * 0.1
            elif leaf == "A_log":
                v = torch.log(0.5 + 3.0 * torch.rand(shape, generator=g))
            elif leaf == "dt_bias":
                v = torch.randn(shape, generator=g) * 0.5 - 1.0
            elif leaf == "D":
                v = 1.0 + torch.randn(shape, generator=g) * 0.1
            elif leaf == "sink":
                v = torch.randn(shape, generator=g)
            elif leaf == "act":
                v = torch.tensor([0.5, 0.5]) + torch.randn(2, generator=g) * 0.1
            elif leaf == "conv":
                v = torch.randn(shape, generator=g) * 0.4
            elif leaf == "b" and len(shape) == 1:
                v = torch.randn(shape, generator=g) * 0.2
            elif name == "embed":
                v = torch.randn(shape, generator=g)
            else:
                v = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            self.weights[name] = v.to(torch.bfloat16)
        self._invalidate()
        return self.to(device) if device is not None else self

    # ---- packing -------------------------------------------------------------------------------
    def _ensure_packed(self):
        if self._packed is not None:
            return self._packed
        dev = self.device
        if dev.type != "cuda":
            raise _lib.EvoError("evo_b200 runs on CUDA (sm_100a) only: move the model with .to('cuda:N'); there is no CPU path")
        w = self.weights
        packed = {"head": _Packed(w["head"]), "layers": []}
        for i, layer in enumerate(self.config.layers):
            p = f"l{i}.mix."
            e = {}
            if layer.kind == "delta":
                # one projection [q | k | v | gate | b | a]; the three convolutions are one over the first 2*qk + vw columns
                e["in"] = _Packed(torch.cat([w[p + n] for n in ("q", "k", "v", "g", "b", "a")], 0))
                e["conv"] = torch.cat([w[p + "q.conv"], w[p + "k.conv"], w[p + "v.conv"]], 0).contiguous()
                e["out"] = _Packed(w[p + "o"])
            else:
                a = layer.left
                # one projection [q | k | v | z | x B C | dt] for the two mixers that read the same input
                e["in"] = _Packed(torch.cat([w[p + "left.q"], w[p + "left.k"], w[p + "left.v"], w[p + "right.in"]], 0))
                e["left_out"], e["right_out"] = _Packed(w[p + "left.o"]), _Packed(w[p + "right.o"])
                if a.rot_dims > 0:
                    half = a.rot_dims // 2
                    f = a.rot_base ** (-2.0 * torch.arange(half, dtype=torch.float64) / a.rot_dims)
                    e["freq"] = f.to(torch.float32).to(dev)
            if layer.ff is not None:
                e["up"], e["down"] = _Packed(w[f"l{i}.mlp.up"]), _Packed(w[f"l{i}.mlp.down"])
            packed["layers"].append(e)
        self._packed = packed
        return packed

    def _cache_tokens(self, key, cache) -> int:
        if key < 0:                                  # pooled rows: one per block of the layer's pool size
            return (cache.shape[1] - 1) * self.config.layers[self.config.runs[-key - 1].layer].left.pool
        return cache.shape[1]

    # ---- kernels ---------------------------------------------------------------------------------
    def _sum_norm(self, x, branches, outs, rows, gather=None):
        """x += sum of the branches (y, ldy, norm weight or None, scale); outs: [(buffer, weight)] normed copies of the new x."""
        cfg = self.config
        p = SumNormParams(x=x.data_ptr(), n_branches=len(branches), eps=cfg.eps, dtype=self._dt, rows=rows, D=cfg.width,
                          gather=gather.data_ptr() if gather is not None else None, ldo=_round_up(cfg.width, 64))
        for b, (y, ldy, nw, scale) in enumerate(branches):
            p.y[b], p.ldy[b], p.norm_w[b], p.scale[b] = y.data_ptr(), ldy, (nw.data_ptr() if nw is not None else None), scale
        for n, (o, wt) in enumerate(outs):
            p.out[n], p.w[n] = o.data_ptr(), wt.data_ptr()
        esz = 4 if self._dt else 2
        nbytes = rows * cfg.width * (8.0 + esz * (len(branches) + len(outs)))
        self._record("sum_norm", nbytes, lambda: check(_lib.lib().evo_sum_norm(C.byref(p), self._stream()), "evo_sum_norm"))

    def _delta(self, r, i, m, h, B, L, rec, fresh):
        y, ld = self._delta_mixer(r, i, m, h, B, L, rec, fresh)
        return [(y, ld, None, 1.0)]

    def _ssd(self, r, i, s, z, col0, ldz, B, L, rec, fresh):
        """z columns [col0, ...) = [gate z | x B C | dt] of the shared projection -> the state-space mixer's output projection."""
        pk = self._packed["layers"][i]
        M, dev = B * L, z.device
        w = self.weights
        esz = z.element_size()
        p = f"l{i}.mix.right."
        inner, gn = s.inner, s.groups * s.state
        base = z.data_ptr() + col0 * esz
        c = self._conv(r, base + inner * esz, ldz, w[p + "conv"], w[p + "conv.b"], s.conv_channels, s.taps, B, L, rec, fresh)
        state, zero = self._matrix_state(r, rec, B, s.heads, s.state, s.vdim, fresh)
        y = torch.empty(M, inner, dtype=torch.float32, device=dev)
        sp = SsdParams(x=c.data_ptr(), Bm=c.data_ptr() + inner * esz, Cm=c.data_ptr() + (inner + gn) * esz, ld=s.conv_channels,
                       dt=base + (2 * inner + 2 * gn) * esz, ld_dt=ldz, A_log=w[p + "A_log"].data_ptr(), dt_bias=w[p + "dt_bias"].data_ptr(),
                       D=w[p + "D"].data_ptr(), state=state.data_ptr(), zero_start=zero, y=y.data_ptr(), dtype=self._dt,
                       B=B, L=L, H=s.heads, G=s.groups, N=s.state, dv=s.vdim)
        self._record("ssd", 3.0 * M * s.heads * s.state * s.vdim, lambda: check(_lib.lib().evo_ssd_fwd(C.byref(sp), self._stream()), "evo_ssd_fwd"))
        ldo = _round_up(inner, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        self._record("gated_group_norm", M * inner * (4.0 + 2.0 * esz), lambda: check(_lib.lib().evo_gated_group_norm(
            ptr(y), C.c_void_p(base), ldz, ptr(w[p + "norm"]), ptr(out), ldo, M, inner, s.norm_groups, self.config.eps, self._dt, self._stream()), "evo_gated_group_norm"))
        return self._linear(out, pk["right_out"], M), pk["right_out"].Np

    def _pooled_rows(self, ip, r, a, cache, B):
        """The pooled-row cache of run r, sized for the token cache it summarises."""
        need = cache.shape[1] // a.pool + 1
        pooled = ip.key_value_memory_dict.get(-(r + 1))
        if pooled is None or pooled.shape[1] < need:
            grown = torch.zeros(cache.shape[0], need, cache.shape[2], dtype=self.act_dtype, device=cache.device)
            if pooled is not None:
                grown[:, :pooled.shape[1]] = pooled
            pooled = ip.key_value_memory_dict[-(r + 1)] = grown
        return pooled

    def _attention(self, r, i, a, z, ldz, B, L, ip, off, pos_dev):
        pk = self._packed["layers"][i]
        M, dev = B * L, z.device
        lib = _lib.lib()
        w = self.weights
        esz = z.element_size()
        p = f"l{i}.mix.left."
        qw, kw, vw = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
        cw = kw + vw
        cache = self._kv_rows(ip, r, cw, B, off, L, pos_dev)
        row, bstride = cw, cache.shape[1] * cw
        qp = QkPrepParams(q=z.data_ptr(), k=z.data_ptr() + qw * esz, v=z.data_ptr() + (qw + kw) * esz, ld=ldz,
                          q_bias=w[p + "q.b"].data_ptr(), k_bias=w[p + "k.b"].data_ptr(), v_bias=w[p + "v.b"].data_ptr(),
                          q_norm_w=w[p + "q.norm"].data_ptr(), k_norm_w=w[p + "k.norm"].data_ptr(), eps=self.config.eps,
                          freq=pk["freq"].data_ptr() if a.rot_dims > 0 else None, rot_dims=a.rot_dims,
                          cache=cache.data_ptr(), cache_row=row, cache_batch_stride=bstride, B=B, L=L, H=a.heads, G=a.kv_heads, dk=a.dim, dv=a.vdim,
                          pos0=off, pos_dev=pos_dev.data_ptr() if pos_dev is not None else None, dtype=self._dt)
        self._record("qk_prep", 2.0 * esz * M * (qw + cw), lambda: check(lib.evo_qk_prep(C.byref(qp), self._stream()), "evo_qk_prep"))
        ldo = _round_up(a.heads * a.vdim, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        ap = WindowAttnParams(q=z.data_ptr(), q_tok_stride=ldz, k=cache.data_ptr(), v=cache.data_ptr() + kw * esz, k_tok_stride=row, v_tok_stride=row,
                              k_batch_stride=bstride, v_batch_stride=bstride, out=out.data_ptr(), ldo=ldo, dtype=self._dt,
                              B=B, Lq=L, H=a.heads, G=a.kv_heads, dk=a.dim, dv=a.vdim, n_maps=1, q_pos0=off,
                              pos_dev=pos_dev.data_ptr() if pos_dev is not None else None, window=a.window, keep_first=0,
                              scale=a.scale, softcap=a.softcap, sink=w[p + "sink"].data_ptr())
        if a.pool > 0:
            pooled = self._pooled_rows(ip, r, a, cache, B)
            check(lib.evo_pool_rows(ptr(cache), row, bstride, ptr(pooled), row, pooled.shape[1] * row, B, L, cw, a.pool, off, ptr(pos_dev), self._dt,
                                    self._stream()), "evo_pool_rows")
            ap.pool, ap.pool_k, ap.pool_v = a.pool, pooled.data_ptr(), pooled.data_ptr() + kw * esz
            ap.pool_tok_stride, ap.pool_batch_stride = row, pooled.shape[1] * row
        span = min(off + L, a.window) if a.window > 0 else off + (L + 1) / 2.0
        if a.pool > 0:
            span += max(0, off + L / 2.0 - a.window) / a.pool
        self._record("window_attn", 4.0 * M * a.heads * span * (a.dim + a.vdim), lambda: check(lib.evo_window_attn_fwd(C.byref(ap), self._stream()), "evo_window_attn_fwd"))
        return self._linear(out, pk["left_out"], M), pk["left_out"].Np

    def _parallel(self, r, i, layer, h, B, L, ip, rec, off, pos_dev, fresh):
        pk = self._packed["layers"][i]
        a = layer.left
        z = self._linear(h, pk["in"], B * L)
        ldz = pk["in"].Np
        left, ldl = self._attention(r, i, a, z, ldz, B, L, ip, off, pos_dev)
        right, ldr = self._ssd(r, i, layer.right, z, a.heads * a.dim + a.kv_heads * (a.dim + a.vdim), ldz, B, L, rec, fresh)
        w = self.weights
        return [(left, ldl, w[f"l{i}.mix.left.out"], 0.5), (right, ldr, w[f"l{i}.mix.right.out"], 0.5)]

    def _feed_forward(self, i, layer, h, M):
        pk = self._packed["layers"][i]
        z = self._linear(h, pk["up"], M)
        a = torch.empty(M, pk["down"].Kp, dtype=self.act_dtype, device=h.device)
        self._record("xielu", 2.0 * z.element_size() * M * layer.ff, lambda: check(_lib.lib().evo_xielu(
            ptr(z), pk["up"].Np, ptr(self.weights[f"l{i}.mlp.act"]), ptr(a), pk["down"].Kp, M, layer.ff, self._dt, self._stream()), "evo_xielu"))
        return (self._linear(a, pk["down"], M), pk["down"].Np, None, 1.0)

    def _body(self, ids, B, L, ipd, off: int, pos_dev=None, rows=None):
        """embed -> every layer -> final norm -> head.  Returns fp32 logits (B*L, V), or (len(rows), V) for the flat row
        indices in `rows` (int64 tensor on the device)."""
        cfg, dev = self.config, ids.device
        lib = _lib.lib()
        M, D, V = B * L, cfg.width, cfg.vocab_size
        if ipd is None:                              # stateless call: the same path on holders that live for this call only
            ipd = self.initialize_inference_params(max_seqlen=L, max_batch_size=B)
        ip, rec = ipd["mha"], ipd["hyena"]
        fresh = pos_dev is None and off == 0         # a sequence's first tokens: recurrent states start from zero
        Kp = _round_up(D, 64)
        x = torch.empty(M, D, dtype=torch.float32, device=dev)
        check(lib.evo_embed_f32(ptr(ids), int(ids.dtype == torch.int64), ptr(self.weights["embed"]), ptr(x), M, D, V, self._stream()), "evo_embed_f32")
        branches = []
        for r, run in enumerate(cfg.runs):
            i = run.layer
            layer = cfg.layers[i]
            h1 = torch.empty(M, Kp, dtype=self.act_dtype, device=dev)
            outs = [(h1, self.weights[f"l{i}.norm1"])]
            if layer.ff is not None:
                h2 = torch.empty(M, Kp, dtype=self.act_dtype, device=dev)
                outs.append((h2, self.weights[f"l{i}.norm2"]))
            self._sum_norm(x, branches, outs, M)
            if self._tap is not None and r > 0:
                self._tap.append(x.clone())
            if layer.kind == "delta":
                branches = self._delta(r, i, layer.delta, h1, B, L, rec, fresh)
            else:
                branches = self._parallel(r, i, layer, h1, B, L, ip, rec, off, pos_dev, fresh)
            if layer.ff is not None:
                branches.append(self._feed_forward(i, layer, h2, M))
        n_out = M if rows is None else int(rows.numel())
        if self._tap is not None:
            self._sum_norm(x, branches, [], M)
            self._tap.append(x.clone())
            branches = []
        if n_out == 0:
            return torch.empty(0, V, dtype=torch.float32, device=dev)
        hf = torch.empty(n_out, Kp, dtype=self.act_dtype, device=dev)
        self._sum_norm(x, branches, [(hf, self.weights["final.norm"])], n_out, gather=rows)
        raw = self._linear(hf, self._packed["head"], n_out)
        logits = torch.empty(n_out, V, dtype=torch.float32, device=dev)
        check(lib.evo_scale_logits(ptr(raw), self._packed["head"].Np, ptr(logits), n_out, V, 1.0, self._dt, self._stream()), "evo_scale_logits")
        return logits
