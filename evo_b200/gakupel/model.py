"""Gakupel: a decoder-only model whose sublayers read the fp32 stream itself and whose OUTPUTS are layer-normed (weight and bias) before
they join it, x <- x + ln1(mixer(x)), x <- x + ln2(ff(x)), and where what a layer hands on is a learned mix of the embedding rows and of
all layers' results so far.  Three kinds of mixer -- causal attention with per-head query / key norms and a partial rotation whose values
are the raw key projections; the gated delta rule; and a pair run side by side on the same input: attention with whole-row norms, a query
temperature, a logarithmic distance bias and a sink in the softmax, beside a matrix memory with exponential gates (mLSTM) -- and two kinds
of feed-forward: dense (erf gelu) and a mixture of experts with sigmoid scores, a choice limited to the best groups of experts, normalised
weights and a gated always-on expert.  Executed by libevo_b200.so.

It follows the object protocol of the framework's other models (see stream_model.StreamDecoder), so the same generation loop, scheduler,
trace replay and command line drive it.  State, keyed by RUN index r:
    d["mha"].key_value_memory_dict[r]   (B, max_seqlen, G*dim + G*vdim): keys (normed, rotated), then values
    d["hyena"].fir_state_dict[r]        (B, taps-1, channels) fp32: the last inputs of the delta rule's short convolutions
    d["hyena"].state_dict[r]            (B, heads, dim, vdim) fp32: the delta rule's matrix state; for the matrix memory
                                        (B, heads, dim, vdim + 1): per head the dim x vdim matrix, then the dim entries of the normaliser
    d["hyena"].state_dict[-(r+1)]       (B, heads) fp32: the matrix memory's running maximum
Closing one sublayer and opening the next is ONE row kernel (evo_post_norm): it sums the sublayer's outputs, norms them into x, after a
feed-forward files the layer's result and mixes the earlier ones, and emits x in the activation type for the next GEMM -- or, for the
last layer, the final norm of the wanted rows.  Linear layers: bf16 activations -> the framework's tcgen05 GEMMs (weights zero-padded once
to their tiles); fp32 activations (dtype=torch.float32) -> evo_gemm_simt, true fp32 multiply-add.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import torch

from .. import _lib
from .._lib import MlstmParams, MoeRouteParams, PostNormParams, QkPrepParams, WindowAttnParams, check, ptr
from ..stream_model import StreamDecoder, _Packed, _round_up
from .config import GakupelConfig

ACT_SILU, ACT_GELU_ERF = 1, 2


class Gakupel(StreamDecoder):
    architecture = "Gakupel"
    gemm_env = "EVO_B200_GAKUPEL_GEMM"

    def __init__(self, config: GakupelConfig, dtype: torch.dtype = torch.bfloat16):
        super().__init__(config, dtype)
        self.fir_taps = max([l.delta.taps for l in config.layers if l.kind == "delta"] or [0])
        # expert mixtures: calls with at least this many rows (outside a captured step) run only the chosen experts, fewer rows run all
        # experts densely with the routing weights multiplied into their columns
        self.moe_sparse_min_rows = int(os.environ.get("EVO_B200_MOE_SPARSE_MIN_ROWS", "1024"))

    # ---- parameters ----------------------------------------------------------------------------
    def init_random(self, seed: int = 0, device=None) -> "Gakupel":
        """Random weights of a usable scale (benchmarks, tests)."""
        g = torch.Generator().manual_seed(seed)
        for name, t in self.weights.items():
            shape = t.shape
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
            if layer.kind == "attention":
                a = layer.attention
                e["in"] = _Packed(torch.cat([w[p + "q"], w[p + "k"]], 0))
                e["out"] = _Packed(w[p + "o"])
            elif layer.kind == "delta":
                # one projection [q | k | v | gate | b | a]; the three convolutions are one over the first 2*qk + vw columns
                e["in"] = _Packed(torch.cat([w[p + n] for n in ("q", "k", "v", "g", "b", "a")], 0))
                e["conv"] = torch.cat([w[p + "q.conv"], w[p + "k.conv"], w[p + "v.conv"]], 0).contiguous()
                e["out"] = _Packed(w[p + "o"])
            else:
                a = layer.attention
                # one projection for the two mixers that read the same input: [q | k | v] of the attention, then [q | k | v | gate | i | f]
                e["in"] = _Packed(torch.cat([w[p + "left." + n] for n in ("q", "k", "v")] + [w[p + "right." + n] for n in ("q", "k", "v", "g", "i", "f")], 0))
                e["left_out"], e["right_out"] = _Packed(w[p + "left.o"]), _Packed(w[p + "right.o"])
                e["sink"] = torch.zeros(a.heads, dtype=torch.bfloat16, device=dev)          # a sink whose score is 0: one more e^0 in the denominator
            if layer.kind != "delta" and layer.attention.rot_dims > 0:
                a = layer.attention
                f = a.rot_base ** (-2.0 * torch.arange(a.rot_dims // 2, dtype=torch.float64) / a.rot_dims)
                e["freq"] = f.to(torch.float32).to(dev)
            f = layer.mlp
            q = f"l{i}.mlp."
            if f is not None and f.kind == "dense":
                e["up"], e["down"] = _Packed(w[q + "up"]), _Packed(w[q + "down"])
            elif f is not None:
                names = [f"e{k}" for k in range(f.experts)] + (["shared"] if f.shared_ff else [])
                e["up"] = _Packed(torch.cat([w[f"{q}{n}.gate"] for n in names] + [w[f"{q}{n}.up"] for n in names], 0))
                e["down"] = _Packed(torch.cat([w[f"{q}{n}.down"] for n in names], 1))
                e["hidden"] = f.experts * f.ff + f.shared_ff
                # the router's rows, then the row of the always-on expert's gate: one fp32 product per token gives all of them
                e["router"] = torch.cat([w[q + "router"]] + ([w[q + "shared.sg"]] if f.shared_ff else []), 0).contiguous()
                e["sparse"] = None                  # per-expert packing, built on the first sparse call
            packed["layers"].append(e)
        self._packed = packed
        return packed

    # ---- kernels ---------------------------------------------------------------------------------
    def _post_norm(self, x, rows, ins=(), norm=None, x_in=None, stack=None, mix_n=0, mix_w=None, out=None, ldo=0, out_norm=None, gather=None):
        """x <- x + ln(sum of ins (y, ldy, scale)) [-> filed in `stack` and mixed] -> out (see evo_post_norm)."""
        cfg = self.config
        w = self.weights
        p = PostNormParams(x=x.data_ptr(), x_in=x_in.data_ptr() if x_in is not None else None, n_in=len(ins), eps=cfg.eps,
                           out=out.data_ptr() if out is not None else None, ldo=ldo, dtype=self._dt, rows=rows, D=cfg.width,
                           gather=gather.data_ptr() if gather is not None else None)
        for b, (y, ldy, scale) in enumerate(ins):
            p.y[b], p.ldy[b], p.scale[b] = y.data_ptr(), ldy, scale
        if norm is not None:
            p.norm_w, p.norm_b = w[norm].data_ptr(), w[norm + ".b"].data_ptr()
        if mix_n:
            p.stack, p.stack_stride, p.mix_n, p.mix_w = stack.data_ptr(), stack.stride(0), mix_n, mix_w.data_ptr()
        if out_norm is not None:
            p.out_norm_w, p.out_norm_b = w[out_norm].data_ptr(), w[out_norm + ".b"].data_ptr()
        esz = 4 if self._dt else 2
        nbytes = rows * cfg.width * (4.0 + (4.0 if ins or mix_n or x_in is not None else 0.0) + esz * (len(ins) + (1 if out is not None else 0)) + 4.0 * mix_n)
        self._record("post_norm", nbytes, lambda: check(_lib.lib().evo_post_norm(C.byref(p), self._stream()), "evo_post_norm"))

    def _attend(self, r, a, z, ldz, cols, norms, per_head, freq, sink, dist, out_pk, B, L, ip, off, pos_dev):
        """Norms / rotation / cache rows (evo_qk_prep), then causal attention over the cache.  cols: columns of q, k, v in z."""
        M, dev, lib = B * L, z.device, _lib.lib()
        esz = z.element_size()
        qw, kw, vw = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
        cw = kw + vw
        cache = self._kv_rows(ip, r, cw, B, off, L, pos_dev)
        row, bstride = cw, cache.shape[1] * cw
        pos_ptr = pos_dev.data_ptr() if pos_dev is not None else None
        qp = QkPrepParams(q=z.data_ptr() + cols[0] * esz, k=z.data_ptr() + cols[1] * esz, v=z.data_ptr() + cols[2] * esz, ld=ldz,
                          q_norm_w=norms[0].data_ptr(), k_norm_w=norms[1].data_ptr(), eps=self.config.eps,
                          freq=freq.data_ptr() if freq is not None else None, rot_dims=a.rot_dims if freq is not None else 0,
                          cache=cache.data_ptr(), cache_row=row, cache_batch_stride=bstride, B=B, L=L, H=a.heads, G=a.kv_heads, dk=a.dim, dv=a.vdim,
                          pos0=off, pos_dev=pos_ptr, dtype=self._dt, norm_per_head=1 if per_head else 0, q_temp_coef=a.q_temp_coef, q_temp_every=a.q_temp_every)
        self._record("qk_prep", 2.0 * esz * M * (qw + cw), lambda: check(lib.evo_qk_prep(C.byref(qp), self._stream()), "evo_qk_prep"))
        ldo = _round_up(a.heads * a.vdim, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        ap = WindowAttnParams(q=z.data_ptr() + cols[0] * esz, q_tok_stride=ldz, k=cache.data_ptr(), v=cache.data_ptr() + kw * esz, k_tok_stride=row, v_tok_stride=row,
                              k_batch_stride=bstride, v_batch_stride=bstride, out=out.data_ptr(), ldo=ldo, dtype=self._dt,
                              B=B, Lq=L, H=a.heads, G=a.kv_heads, dk=a.dim, dv=a.vdim, n_maps=1, q_pos0=off, pos_dev=pos_ptr, window=0, keep_first=0,
                              scale=a.scale, sink=sink.data_ptr() if sink is not None else None,
                              dist_r1=dist[0].data_ptr() if dist is not None else None, dist_r2=dist[1].data_ptr() if dist is not None else None)
        span = off + (L + 1) / 2.0
        self._record("window_attn", 4.0 * M * a.heads * span * (a.dim + a.vdim), lambda: check(lib.evo_window_attn_fwd(C.byref(ap), self._stream()), "evo_window_attn_fwd"))
        return self._linear(out, out_pk, M), out_pk.Np

    def _attention(self, r, i, a, h, B, L, ip, off, pos_dev):
        pk = self._packed["layers"][i]
        w, p = self.weights, f"l{i}.mix."
        z = self._linear(h, pk["in"], B * L)
        qw = a.heads * a.dim
        # the values are the key projections as they leave the GEMM: the value columns are the key columns
        y, ld = self._attend(r, a, z, pk["in"].Np, (0, qw, qw), (w[p + "q.norm"], w[p + "k.norm"]), True, pk.get("freq"), None, None, pk["out"], B, L, ip, off, pos_dev)
        return [(y, ld, 1.0)]

    def _memory(self, r, i, s, z, col0, ldz, B, L, rec, fresh):
        """z columns [col0, ...) = [q | k | v | gate | i | f] of the shared projection -> the matrix memory's output projection."""
        pk = self._packed["layers"][i]
        M, dev, w = B * L, z.device, self.weights
        esz = z.element_size()
        p = f"l{i}.mix.right."
        qk, vw = s.heads * s.dim, s.heads * s.vdim
        base = z.data_ptr() + col0 * esz
        state, zero = self._matrix_state(r, rec, B, s.heads, s.dim, s.vdim + 1, fresh)
        mrun = rec.state_dict.get(-(r + 1))
        if mrun is None:
            mrun = rec.state_dict[-(r + 1)] = torch.zeros(B, s.heads, dtype=torch.float32, device=dev)
        ldo = _round_up(vw, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        mp = MlstmParams(q=base, k=base + qk * esz, v=base + 2 * qk * esz, ld=ldz, gi=base + (2 * qk + 2 * vw) * esz, gf=base + (2 * qk + 2 * vw + s.heads) * esz, ldg=ldz,
                         i_bias=w[p + "i.b"].data_ptr(), f_bias=w[p + "f.b"].data_ptr(), cap=s.gate_cap, q_scale=s.dim ** -0.5, den_eps=1e-6,
                         gate=base + (2 * qk + vw) * esz, ld_gate=ldz, norm_w=w[p + "norm"].data_ptr(), eps=self.config.eps,
                         state=state.data_ptr(), mstate=mrun.data_ptr(), zero_start=zero, out=out.data_ptr(), ldo=ldo, dtype=self._dt,
                         B=B, L=L, H=s.heads, dk=s.dim, dv=s.vdim)
        nws = _lib.lib().evo_mlstm_workspace(C.byref(mp))
        ws = torch.empty(nws, dtype=torch.uint8, device=dev) if nws else None
        self._record("mlstm", 3.0 * M * s.heads * s.dim * s.vdim, lambda: check(_lib.lib().evo_mlstm_fwd(C.byref(mp), ptr(ws), nws, self._stream()), "evo_mlstm_fwd"))
        return self._linear(out, pk["right_out"], M), pk["right_out"].Np

    def _parallel(self, r, i, layer, h, B, L, ip, rec, off, pos_dev, fresh):
        pk = self._packed["layers"][i]
        a, w, p = layer.attention, self.weights, f"l{i}.mix.left."
        z = self._linear(h, pk["in"], B * L)
        ldz = pk["in"].Np
        qw, kw, vw = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
        left, ldl = self._attend(r, a, z, ldz, (0, qw, qw + kw), (w[p + "q.norm"], w[p + "k.norm"]), False, pk.get("freq"), pk["sink"],
                                 (w[p + "r1"], w[p + "r2"]), pk["left_out"], B, L, ip, off, pos_dev)
        right, ldr = self._memory(r, i, layer.memory, z, qw + kw + vw, ldz, B, L, rec, fresh)
        return [(left, ldl, layer.left_scale), (right, ldr, layer.right_scale)]

    def _route(self, i, f, h, M, chosen=None):
        """Routing weights (M, experts [+ 1: the always-on expert's gate]) fp32 from the stream's rows h."""
        pk = self._packed["layers"][i]
        n_extra = 1 if f.shared_ff else 0
        route = torch.empty(M, f.experts + n_extra, dtype=torch.float32, device=h.device)
        rp = MoeRouteParams(h=h.data_ptr(), ldh=h.shape[1], router_w=pk["router"].data_ptr(), correction=self.weights[f"l{i}.mlp.correction"].data_ptr(),
                            weights=route.data_ptr(), ldw=f.experts + n_extra, chosen=chosen.data_ptr() if chosen is not None else None,
                            rows=M, D=self.config.width, E=f.experts, top=f.top, n_extra=n_extra, score_fn=1, groups=f.groups, keep=f.keep,
                            normalize=1, norm_eps=1e-20, scale=f.router_scale, dtype=self._dt)
        self._record("moe_route", float(M) * self.config.width * h.element_size(), lambda: check(_lib.lib().evo_moe_route_ex(C.byref(rp), self._stream()), "evo_moe_route"))
        return route

    def _experts_sparse(self, i, f, h, M):
        """Only the chosen experts (see StreamDecoder._run_chosen_experts), then the weighted sum per token on top of the gated always-on expert."""
        pk = self._packed["layers"][i]
        dev, w, lib, D, q = h.device, self.weights, _lib.lib(), self.config.width, f"l{i}.mlp."
        if pk["sparse"] is None:
            sp = {"experts": [(_Packed(torch.cat([w[f"{q}e{k}.gate"], w[f"{q}e{k}.up"]], 0)), _Packed(w[f"{q}e{k}.down"])) for k in range(f.experts)]}
            if f.shared_ff:
                sp["shared_up"], sp["shared_down"] = _Packed(torch.cat([w[q + "shared.gate"], w[q + "shared.up"]], 0)), _Packed(w[q + "shared.down"])
            pk["sparse"] = sp
        sp = pk["sparse"]
        E, top, esz = f.experts, f.top, h.element_size()
        chosen = torch.full((M, top), -1, dtype=torch.int32, device=dev)
        route = self._route(i, f, h, M, chosen)
        ys, slot_of = self._run_chosen_experts(h, M, chosen, sp["experts"], f.ff, E, top)
        base, ldb = None, 0
        if f.shared_ff:
            su, sd = sp["shared_up"], sp["shared_down"]
            zr = self._linear(h, su, M)
            a = torch.empty(M, sd.Kp, dtype=self.act_dtype, device=dev)
            self._record("glu_act", 3.0 * esz * M * f.shared_ff, lambda: check(lib.evo_glu_act(
                ptr(zr), C.c_void_p(zr.data_ptr() + f.shared_ff * esz), su.Np, ptr(a), sd.Kp, M, f.shared_ff, ACT_SILU, None, 0, 0, 0, 0, self._dt, self._stream()), "evo_glu_act"))
            base, ldb = self._linear(a, sd, M), sd.Np
        ldo = _round_up(D, 64)
        y = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        self._record("moe_combine", float(M) * D * esz * (2.0 + top), lambda: check(lib.evo_moe_combine(
            ptr(ys), sp["experts"][0][1].Np, ptr(base), ldb, ptr(route), route.shape[1], 1 if f.shared_ff else 0, ptr(chosen), ptr(slot_of), ptr(y), ldo,
            M, D, E, top, self._dt, self._stream()), "evo_moe_combine"))
        return y, ldo

    def _feed_forward(self, i, f, h, M, captured=False):
        pk = self._packed["layers"][i]
        dev, lib = h.device, _lib.lib()
        if f.kind == "moe" and not captured and M >= self.moe_sparse_min_rows and f.top < f.experts:
            return self._experts_sparse(i, f, h, M)
        z = self._linear(h, pk["up"], M)
        esz, ld = z.element_size(), pk["up"].Np
        a = torch.empty(M, pk["down"].Kp, dtype=self.act_dtype, device=dev)
        if f.kind == "dense":
            self._record("act", 2.0 * esz * M * f.ff, lambda: check(lib.evo_glu_act(
                ptr(z), None, ld, ptr(a), pk["down"].Kp, M, f.ff, ACT_GELU_ERF, None, 0, 0, 0, 0, self._dt, self._stream()), "evo_glu_act"))
        else:
            # all experts densely: the routing weights (0 for experts that were not chosen) and the always-on expert's gate multiply the
            # experts' columns, and the weighted sum over experts is the K-reduction of one down GEMM
            F = pk["hidden"]
            route = self._route(i, f, h, M)
            self._record("glu_act", 3.0 * esz * M * F, lambda: check(lib.evo_glu_act(
                ptr(z), C.c_void_p(z.data_ptr() + F * esz), ld, ptr(a), pk["down"].Kp, M, F, ACT_SILU, ptr(route), route.shape[1], f.ff, f.experts,
                1 if f.shared_ff else 0, self._dt, self._stream()), "evo_glu_act"))
        return self._linear(a, pk["down"], M), pk["down"].Np

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
        n_layers = len(cfg.runs)
        n_out = M if rows is None else int(rows.numel())
        # slot 0: the embedding rows, slot j: the result of layer j - 1 -- what every layer's mix reads
        stack = torch.empty(n_layers + 1, M, D, dtype=torch.float32, device=dev)
        check(lib.evo_embed_f32(ptr(ids), int(ids.dtype == torch.int64), ptr(self.weights["embed"]), ptr(stack), M, D, V, self._stream()), "evo_embed_f32")
        x = torch.empty(M, D, dtype=torch.float32, device=dev)
        h = torch.empty(M, Kp, dtype=self.act_dtype, device=dev)
        self._post_norm(x, M, x_in=stack[0], out=h, ldo=Kp)
        hf = None
        for r, run in enumerate(cfg.runs):
            i = run.layer
            layer = cfg.layers[i]
            if layer.kind == "attention":
                ins = self._attention(r, i, layer.attention, h, B, L, ip, off, pos_dev)
            elif layer.kind == "delta":
                y, ld = self._delta_mixer(r, i, layer.delta, h, B, L, rec, fresh)
                ins = [(y, ld, 1.0)]
            else:
                ins = self._parallel(r, i, layer, h, B, L, ip, rec, off, pos_dev, fresh)
            norm = f"l{i}.norm1"
            if layer.mlp is not None:
                h = torch.empty(M, Kp, dtype=self.act_dtype, device=dev)
                self._post_norm(x, M, ins, norm, out=h, ldo=Kp)
                y, ld = self._feed_forward(i, layer.mlp, h, M, captured=pos_dev is not None)
                ins, norm = [(y, ld, 1.0)], f"l{i}.norm2"
            mix = dict(stack=stack, mix_n=r + 2, mix_w=self.weights[f"l{i}.dwa"])
            if r + 1 < n_layers or self._tap is not None:
                h = torch.empty(M, Kp, dtype=self.act_dtype, device=dev)
                self._post_norm(x, M, ins, norm, out=h, ldo=Kp, **mix)
                if self._tap is not None:
                    self._tap.append(x.clone())
            elif n_out:                              # the last layer closes on the wanted rows only, with the final norm
                hf = torch.empty(n_out, Kp, dtype=self.act_dtype, device=dev)
                self._post_norm(x, n_out, ins, norm, out=hf, ldo=Kp, out_norm="final.norm", gather=rows, **mix)
        if n_out == 0:
            return torch.empty(0, V, dtype=torch.float32, device=dev)
        if hf is None:
            hf = torch.empty(n_out, Kp, dtype=self.act_dtype, device=dev)
            self._post_norm(x, n_out, out=hf, ldo=Kp, out_norm="final.norm", gather=rows)
        raw = self._linear(hf, self._packed["head"], n_out)
        logits = torch.empty(n_out, V, dtype=torch.float32, device=dev)
        check(lib.evo_scale_logits(ptr(raw), self._packed["head"].Np, ptr(logits), n_out, V, 1.0, self._dt, self._stream()), "evo_scale_logits")
        return logits
