"""Movalorn: a decoder-only model with an fp32 residual stream whose branches are normed on both sides (one-number RMS gains) and
gated by a sigmoid of the branch input, a token + hashed-pair embedding, two kinds of mixer (latent attention with a shared
rotated key part, a sliding window and one output gate per head; the minGRU element-wise recurrence), two kinds of
feed-forward (gated dense; routed experts plus an always-on expert) and a weight-shared loop over a span of layers that
re-projects [stream ; embedding output] before every pass -- executed by libevo_b200.so.

The class is a StreamDecoder: forward protocol, state holders, trace replay and the on-device generation loop are the shared ones.
State (keyed by RUN index, a looped layer has one entry per pass):
    d["mha"].key_value_memory_dict[r]   (B, max_seqlen, row) latent cache: [latent | 0.. | rotated key part | 0..], activation dtype
    d["hyena"].state_dict[r]            (B, width) fp32: the minGRU state
    d["hyena"].state_dict[-1]           (B,) int64: each sequence's last token (-1: none yet) for the pair embedding
Per layer, with n(u; g) = u / sqrt(mean(u^2) + eps) * g:
    h = n(x; g1);  x += n(mixer(h) * sigmoid(R1 h + r1); g1b);   h = n(x; g2);  x += n(ff(h) * sigmoid(R2 h + r2); g2b)
Closing one branch and opening the next is ONE row kernel (evo_branch_norm), so x is read and written once per branch; the gate
projections R ride in the branch's input GEMM.  Linear layers: bf16 activations -> the tcgen05 GEMMs; fp32 activations
(dtype=torch.float32) -> evo_gemm_simt.  Routed experts are computed densely: one GEMM against all experts' [gate ; up] rows, the
activation kernel multiplies each expert's columns by the token's routing weight (0 when not chosen), and the weighted sum over
experts is the K-reduction of one down GEMM against the experts' concatenated down weights.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

from .. import _lib
from .._lib import BranchNormParams, LatentDecodeParams, LatentPrepParams, MinGruParams, WindowAttnParams, check, ptr
from ..stream_model import StreamDecoder, _Packed, _round_up
from ..stripedhyena.cache import InferenceParams, RecurrentInferenceParams
from .config import MovalornConfig

PREV_TOKEN = -1               # key of the last-token vector in the recurrent state holder
ABSORBED_MAX_ROWS = 4         # portions up to this many tokens attend straight from the latent cache


class _Pending:
    """A finished branch whose result is not yet in the stream: y (+ its gate) is folded in by the next evo_branch_norm."""

    def __init__(self, y, ldy, gate_ptr=None, ldg=0, gate_bias=None, post_gain=None, replace=False, row_add=None, hold=None):
        self.y, self.ldy, self.gate_ptr, self.ldg, self.gate_bias = y, ldy, gate_ptr, ldg, gate_bias
        self.post_gain, self.replace, self.row_add = post_gain, replace, row_add
        self.hold = hold          # the buffer gate_ptr points into: alive until the folding kernel is launched


class Movalorn(StreamDecoder):
    architecture = "Movalorn"
    gemm_env = "EVO_B200_MOVALORN_GEMM"

    def __init__(self, config: MovalornConfig, dtype: torch.dtype = torch.bfloat16):
        super().__init__(config, dtype)
        # few-row latent attention: "shared" = heads share each tile of latents (three launches), "head" = one CTA per (query, head)
        self.latent_decode_path = os.environ.get("EVO_B200_LATENT_DECODE", "shared")
        # expert mixtures: calls with at least this many rows (outside a captured step) run only the chosen experts, one GEMM pair per
        # expert over the rows sorted by expert (the per-expert row counts come back to the host); fewer rows run all experts densely
        self.moe_sparse_min_rows = int(os.environ.get("EVO_B200_MOE_SPARSE_MIN_ROWS", "1024"))

    # ---- parameters ----------------------------------------------------------------------------
    def init_random(self, seed: int = 0, device=None) -> "Movalorn":
        """Random weights of a usable scale (benchmarks, tests)."""
        g = torch.Generator().manual_seed(seed)
        for name, t in self.weights.items():
            shape = t.shape
            leaf = name.split(".")[-1]
            if leaf in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
                v = 0.5 + torch.rand(shape, generator=g)
            elif name.endswith("dkv.norm"):
                v = 1.0 + torch.randn(shape, generator=g) * 0.1
            elif leaf == "b" or leaf == "correction":
                v = torch.randn(shape, generator=g) * 0.3
            elif name == "embed":
                v = torch.randn(shape, generator=g) / max(self.config.embed_scale, 1e-6)
            elif name in ("bigram", "loop.step"):
                v = torch.randn(shape, generator=g) * 0.3
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
        cfg, w = self.config, self.weights
        scalars = {k: float(v.float()) for k, v in w.items() if v.dim() == 0}
        packed = {"head": _Packed(w["head"]), "layers": [], "gain": scalars}
        if cfg.looped:
            packed["loop_in"] = _Packed(w["loop.in"])
        for i, layer in enumerate(cfg.layers):
            m, f, p = layer.mixer, layer.mlp, f"l{i}."
            e = {}
            if m.kind == "mingru":
                e["in"] = _Packed(torch.cat([w[p + "mix.z"], w[p + "mix.x"], w[p + "mix.g"], w[p + "rg1"]], 0))
            else:
                e["in"] = _Packed(torch.cat([w[p + "mix.q"], w[p + "mix.dkv"], w[p + "mix.g"], w[p + "rg1"]], 0))
                # expansion of cache rows [latent | 0.. | rotated key part] into per-head keys [Uk_h c | rotated part] and values Uv_h c:
                # identity rows carry the shared rotated part into every head's key
                rank_pad = _round_up(m.kv_rank, 8)
                hd = m.dim + m.rot_dim
                up = torch.zeros(m.heads * hd + m.heads * m.vdim, rank_pad + m.rot_dim, dtype=torch.bfloat16, device=dev)
                for h in range(m.heads):
                    up[h * hd:h * hd + m.dim, :m.kv_rank] = w[p + "mix.uk"][h * m.dim:(h + 1) * m.dim]
                    up[h * hd + m.dim:(h + 1) * hd, rank_pad:] = torch.eye(m.rot_dim, dtype=torch.bfloat16, device=dev)
                up[m.heads * hd:, :m.kv_rank] = w[p + "mix.uv"]
                e["expand"] = _Packed(up)
                e["rank_pad"] = rank_pad
                e["cache_row"] = e["expand"].Kp
                i2 = torch.arange(0, m.rot_dims, 2, dtype=torch.float32)
                e["freq"] = (torch.tensor(m.rot_base, dtype=torch.float32) ** (-i2 / m.rot_dims)).to(dev) if m.rot_dims else torch.zeros(1, device=dev)
            e["out"] = _Packed(w[p + "mix.o"])
            if f is not None and f.kind == "dense":
                e["up"] = _Packed(torch.cat([w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "rg2"]], 0))
                e["down"] = _Packed(w[p + "mlp.down"])
                e["hidden"] = f.ff
            elif f is not None:
                names = [f"e{k}" for k in range(f.experts)] + (["shared"] if f.shared_ff else [])
                e["up"] = _Packed(torch.cat([w[f"{p}mlp.{n}.gate"] for n in names] + [w[f"{p}mlp.{n}.up"] for n in names] + [w[p + "rg2"]], 0))
                e["down"] = _Packed(torch.cat([w[f"{p}mlp.{n}.down"] for n in names], 1))
                e["hidden"] = f.experts * f.ff + f.shared_ff
                e["sparse"] = None                  # per-expert packing, built on the first sparse call
            packed["layers"].append(e)
        self._packed = packed
        return packed

    # ---- kernels ---------------------------------------------------------------------------------
    def _branch_norm(self, x, pend: Optional[_Pending], gain: float, out=None, ldo=0, rows=None, concat=None, gather=None):
        cfg = self.config
        n = int(gather.numel()) if gather is not None else (x.shape[0] if rows is None else rows)
        p = BranchNormParams(x=x.data_ptr(), gain=gain, eps=cfg.eps, out=out.data_ptr() if out is not None else None, ldo=ldo,
                             concat=1 if concat is not None else 0, cat=concat.data_ptr() if concat is not None else None,
                             dtype=self._dt, rows=n, D=cfg.width, gather=gather.data_ptr() if gather is not None else None)
        if pend is not None:
            p.y, p.ldy = pend.y.data_ptr(), pend.ldy
            if pend.gate_ptr is not None:
                p.gate, p.ldg, p.gate_bias = pend.gate_ptr, pend.ldg, pend.gate_bias.data_ptr()
            if pend.post_gain is not None:
                p.post_norm, p.post_gain = 1, pend.post_gain
            p.replace = 1 if pend.replace else 0
            p.row_add = pend.row_add.data_ptr() if pend.row_add is not None else None
        esz = 4 if self._dt else 2
        nbytes = n * cfg.width * ((8.0 if pend is not None else 4.0) + (2.0 * esz if pend is not None else 0.0) + (esz if out is not None else 0.0))
        self._record("branch_norm", nbytes, lambda: check(_lib.lib().evo_branch_norm(C.byref(p), self._stream()), "evo_branch_norm"))

    def _open(self, x, pend, gain, M):
        """Fold the pending branch into the stream and return norm(x) * gain as (M, Kp) GEMM input."""
        Kp = _round_up(self.config.width, 64)
        h = torch.empty(M, Kp, dtype=self.act_dtype, device=x.device)
        self._branch_norm(x, pend, gain, out=h, ldo=Kp)
        return h

    def _mingru(self, r, i, m, h, B, L, rec: Optional[RecurrentInferenceParams]):
        pk = self._packed["layers"][i]
        M, dev, w = B * L, h.device, self.weights
        z = self._linear(h, pk["in"], M)
        esz, W, ld = z.element_size(), m.width, pk["in"].Np
        ldo = _round_up(W, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        state, zero = None, 1
        if rec is not None:
            state = rec.state_dict.get(r)
            zero = 0
            if state is None:
                state = rec.state_dict[r] = torch.zeros(B, W, dtype=torch.float32, device=dev)
        gp = MinGruParams(z=z.data_ptr(), u=z.data_ptr() + W * esz, g=z.data_ptr() + 2 * W * esz, ld=ld,
                          z_bias=w[f"l{i}.mix.z.b"].data_ptr(), u_bias=w[f"l{i}.mix.x.b"].data_ptr(),
                          state=state.data_ptr() if state is not None else None, zero_start=zero,
                          out=out.data_ptr(), ldo=ldo, dtype=self._dt, B=B, L=L, W=W)
        nws = _lib.lib().evo_mingru_workspace(C.byref(gp))
        ws = torch.empty(nws, dtype=torch.uint8, device=dev) if nws else None
        self._record("mingru", float(M) * W * esz * (4.0 + (2.0 if nws else 0.0)),
                     lambda: check(_lib.lib().evo_mingru_fwd(C.byref(gp), ptr(ws), nws, self._stream()), "evo_mingru_fwd"))
        y = self._linear(out, pk["out"], M)
        return _Pending(y, pk["out"].Np, z.data_ptr() + 3 * W * esz, ld, w[f"l{i}.rg1.b"], self._packed["gain"][f"l{i}.norm1b"], hold=z)

    def _latent_attention(self, r, i, m, h, B, L, ip: Optional[InferenceParams], off: int, pos_dev):
        pk = self._packed["layers"][i]
        M, dev, w, lib = B * L, h.device, self.weights, _lib.lib()
        z = self._linear(h, pk["in"], M)
        esz, ld = z.element_size(), pk["in"].Np
        hd = m.dim + m.rot_dim
        qw, aw = m.heads * hd, m.kv_rank + m.rot_dim
        rank_pad, cache_row = pk["rank_pad"], pk["cache_row"]
        if ip is None:
            cache = torch.zeros(B, L, cache_row, dtype=self.act_dtype, device=dev)
        else:
            cache = self._kv_rows(ip, r, cache_row, B, off, L, pos_dev)
        bstride = cache.shape[1] * cache_row
        pos_ptr = pos_dev.data_ptr() if pos_dev is not None else None
        pp = LatentPrepParams(q=z.data_ptr(), ldq=ld, dkv=z.data_ptr() + qw * esz, ld_dkv=ld, norm_w=w[f"l{i}.mix.dkv.norm"].data_ptr(), eps=self.config.eps,
                              freq=pk["freq"].data_ptr(), cache=cache.data_ptr(), cache_row=cache_row, cache_batch_stride=bstride, rank_pad=rank_pad,
                              B=B, L=L, H=m.heads, dim=m.dim, rot=m.rot_dim, rank=m.kv_rank, pos0=off, pos_dev=pos_ptr, dtype=self._dt, rot_dims=m.rot_dims)
        self._record("latent_prep", float(M) * (qw + 2 * aw) * esz, lambda: check(lib.evo_latent_prep(C.byref(pp), self._stream()), "evo_latent_prep"))
        inner = m.heads * m.vdim
        ldo = _round_up(inner, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        gate_ptr = z.data_ptr() + (qw + aw) * esz
        span = min(off + L, m.window) if m.window > 0 else off + (L + 1) / 2.0
        if L <= ABSORBED_MAX_ROWS or pos_dev is not None:
            dp = LatentDecodeParams(q=z.data_ptr(), ldq=ld, cache=cache.data_ptr(), cache_row=cache_row, cache_batch_stride=bstride, rank_pad=rank_pad,
                                    uk=w[f"l{i}.mix.uk"].data_ptr(), uv=w[f"l{i}.mix.uv"].data_ptr(), gate=gate_ptr, ld_gate=ld,
                                    out=out.data_ptr(), ldo=ldo, B=B, Lq=L, H=m.heads, dim=m.dim, rot=m.rot_dim, rank=m.kv_rank, vdim=m.vdim,
                                    pos0=off, pos_dev=pos_ptr, window=m.window, scale=m.scale, dtype=self._dt,
                                    max_keys=cache.shape[1] if pos_dev is not None else off + L)
            nws = lib.evo_latent_attn_decode_workspace(C.byref(dp)) if self.latent_decode_path == "shared" else 0
            ws = torch.empty(nws, dtype=torch.uint8, device=dev) if nws else None
            # roofline bytes: each sequence's visible latents once (all heads share them)
            self._record("latent_decode", float(M) * span * (m.kv_rank + m.rot_dim) * esz,
                         lambda: check(lib.evo_latent_attn_decode(C.byref(dp), ptr(ws), nws, self._stream()), "evo_latent_attn_decode"))
        else:
            lo = max(0, off - (m.window - 1)) if m.window > 0 else 0
            n = off + L - lo
            ex = pk["expand"]
            kv = torch.empty(B, n, ex.Np, dtype=self.act_dtype, device=dev)
            for b in range(B):
                self._linear(cache[b, lo:off + L], ex, n, out=kv[b])
            ap = WindowAttnParams(q=z.data_ptr(), q_tok_stride=ld, gate=gate_ptr, gate_tok_stride=ld, gate_per_head=1,
                                  k=kv.data_ptr() - lo * ex.Np * esz, v=kv.data_ptr() + (qw - lo * ex.Np) * esz,
                                  k_tok_stride=ex.Np, v_tok_stride=ex.Np, k_batch_stride=n * ex.Np, v_batch_stride=n * ex.Np,
                                  out=out.data_ptr(), ldo=ldo, dtype=self._dt, B=B, Lq=L, H=m.heads, G=m.heads, dk=hd, dv=m.vdim, n_maps=1,
                                  q_pos0=off, pos_dev=None, window=m.window, keep_first=0, scale=m.scale, lambda_=0.0, head_norm=0,
                                  norm_eps=self.config.eps, out_scale=1.0)
            self._record("window_attn", 4.0 * M * m.heads * span * (hd + m.vdim),
                         lambda: check(lib.evo_window_attn_fwd(C.byref(ap), self._stream()), "evo_window_attn_fwd"))
        y = self._linear(out, pk["out"], M)
        return _Pending(y, pk["out"].Np, z.data_ptr() + (qw + aw + m.heads) * esz, ld, w[f"l{i}.rg1.b"], self._packed["gain"][f"l{i}.norm1b"], hold=z)

    def _sparse_pack(self, i, f):
        pk = self._packed["layers"][i]
        if pk["sparse"] is None:
            w, p = self.weights, f"l{i}.mlp."
            sp = {"experts": [(_Packed(torch.cat([w[f"{p}e{k}.gate"], w[f"{p}e{k}.up"]], 0)), _Packed(w[f"{p}e{k}.down"])) for k in range(f.experts)]}
            rest = ([w[p + "shared.gate"], w[p + "shared.up"]] if f.shared_ff else []) + [w[f"l{i}.rg2"]]
            sp["rest"] = _Packed(torch.cat(rest, 0))
            sp["shared_down"] = _Packed(w[p + "shared.down"]) if f.shared_ff else None
            pk["sparse"] = sp
        return pk["sparse"]

    def _experts_sparse(self, i, f, h, M):
        """Only the chosen experts: route, sort the (token, choice) pairs by expert, one [gate ; up] GEMM, activation and down GEMM per
        expert over its slice, then the weighted sum per token on top of the always-on expert."""
        sp = self._sparse_pack(i, f)
        dev, w, lib, D = h.device, self.weights, _lib.lib(), self.config.width
        E, top, n = f.experts, f.top, M * f.top
        esz = h.element_size()
        route = torch.empty(M, E, dtype=torch.float32, device=dev)
        chosen = torch.full((M, top), -1, dtype=torch.int32, device=dev)
        self._record("moe_route", float(M) * D * esz, lambda: check(lib.evo_moe_route(
            ptr(h), h.shape[1], ptr(w[f"l{i}.mlp.router"]), ptr(w[f"l{i}.mlp.correction"]), ptr(route), ptr(chosen), M, D,
            E, top, f.router_scale, self._dt, self._stream()), "evo_moe_route"))
        ys, slot_of = self._run_chosen_experts(h, M, chosen, sp["experts"], f.ff, E, top)
        down0 = sp["experts"][0][1]
        # the always-on expert and the branch gate read every row
        rest = sp["rest"]
        zr = self._linear(h, rest, M)
        base, ldb = None, 0
        if f.shared_ff:
            sd = sp["shared_down"]
            a = torch.empty(M, sd.Kp, dtype=self.act_dtype, device=dev)
            self._record("glu_act", 3.0 * esz * M * f.shared_ff, lambda: check(lib.evo_glu_act(
                ptr(zr), C.c_void_p(zr.data_ptr() + f.shared_ff * esz), rest.Np, ptr(a), sd.Kp, M, f.shared_ff, 1, None, 0, 0, 0, 0, self._dt, self._stream()), "evo_glu_act"))
            base = self._linear(a, sd, M)
            ldb = sd.Np
        ldo = _round_up(D, 64)
        y = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        self._record("moe_combine", float(M) * D * esz * (2.0 + top), lambda: check(lib.evo_moe_combine(
            ptr(ys), down0.Np, ptr(base), ldb, ptr(route), E, 0, ptr(chosen), ptr(slot_of), ptr(y), ldo, M, D, E, top, self._dt, self._stream()), "evo_moe_combine"))
        return _Pending(y, ldo, zr.data_ptr() + 2 * f.shared_ff * esz, rest.Np, w[f"l{i}.rg2.b"], self._packed["gain"][f"l{i}.norm2b"], hold=zr)

    def _feed_forward(self, i, f, h, M, captured=False):
        pk = self._packed["layers"][i]
        dev, w, lib = h.device, self.weights, _lib.lib()
        if f.kind == "moe" and not captured and M >= self.moe_sparse_min_rows and f.top < f.experts:
            return self._experts_sparse(i, f, h, M)
        z = self._linear(h, pk["up"], M)
        esz, ld, F = z.element_size(), pk["up"].Np, pk["hidden"]
        a = torch.empty(M, pk["down"].Kp, dtype=self.act_dtype, device=dev)
        route = None
        if f.kind == "moe":
            route = torch.empty(M, f.experts, dtype=torch.float32, device=dev)
            self._record("moe_route", float(M) * self.config.width * esz, lambda: check(lib.evo_moe_route(
                ptr(h), h.shape[1], ptr(w[f"l{i}.mlp.router"]), ptr(w[f"l{i}.mlp.correction"]), ptr(route), None, M, self.config.width,
                f.experts, f.top, f.router_scale, self._dt, self._stream()), "evo_moe_route"))
        self._record("glu_act", 3.0 * esz * M * F, lambda: check(lib.evo_glu_act(
            ptr(z), C.c_void_p(z.data_ptr() + F * esz), ld, ptr(a), pk["down"].Kp, M, F, 0 if f.kind == "dense" else 1,
            ptr(route), f.experts if route is not None else 0, f.ff if route is not None else 0, f.experts if route is not None else 0, 0, self._dt, self._stream()), "evo_glu_act"))
        y = self._linear(a, pk["down"], M)
        return _Pending(y, pk["down"].Np, z.data_ptr() + 2 * F * esz, ld, w[f"l{i}.rg2.b"], self._packed["gain"][f"l{i}.norm2b"], hold=z)

    def _body(self, ids, B, L, ipd, off: int, pos_dev=None, rows=None):
        """embedding -> every run -> final norm -> head -> logit scale.  Returns fp32 logits (B*L, V), or (len(rows), V) for the
        flat row indices in `rows` (int64 tensor on the device)."""
        cfg, dev, lib = self.config, ids.device, _lib.lib()
        M, D, V = B * L, cfg.width, cfg.vocab_size
        gain = self._packed["gain"]
        ip = ipd["mha"] if ipd is not None else None
        rec = ipd["hyena"] if ipd is not None else None
        prev = None
        if rec is not None:
            prev = rec.state_dict.get(PREV_TOKEN)
            if prev is None:
                prev = rec.state_dict[PREV_TOKEN] = torch.full((B,), -1, dtype=torch.int64, device=dev)
        x = torch.empty(M, D, dtype=torch.float32, device=dev)
        check(lib.evo_embed_pair_f32(ptr(ids), int(ids.dtype == torch.int64), ptr(self.weights["embed"]), ptr(self.weights["bigram"]), ptr(x), ptr(prev),
                                     B, L, D, V, cfg.embed_scale, cfg.buckets, cfg.mul_prev, cfg.mul_cur, self._stream()), "evo_embed_pair_f32")
        x0 = x.clone() if cfg.looped else None
        pend = None
        for r, run in enumerate(cfg.runs):
            layer = cfg.layers[run.layer]
            m, p = layer.mixer, f"l{run.layer}."
            if run.first:
                K2 = self._packed["loop_in"].Kp
                cat = torch.empty(M, K2, dtype=self.act_dtype, device=dev)
                self._branch_norm(x, pend, 1.0, out=cat, ldo=K2, concat=x0)
                y = self._linear(cat, self._packed["loop_in"], M)
                pend = _Pending(y, self._packed["loop_in"].Np, replace=True, row_add=self.weights["loop.step"][run.loop_pass])
            h = self._open(x, pend, gain[p + "norm1"], M)
            if m.kind == "mingru":
                pend = self._mingru(r, run.layer, m, h, B, L, rec)
            else:
                pend = self._latent_attention(r, run.layer, m, h, B, L, ip, off, pos_dev)
            if layer.mlp is not None:
                h = self._open(x, pend, gain[p + "norm2"], M)
                pend = self._feed_forward(run.layer, layer.mlp, h, M, captured=pos_dev is not None)
            if self._tap is not None:
                self._branch_norm(x, pend, 1.0)
                pend = None
                self._tap.append(x.clone())
        n_out = M if rows is None else int(rows.numel())
        if n_out == 0:
            return torch.empty(0, V, dtype=torch.float32, device=dev)
        Kp = _round_up(D, 64)
        hf = torch.empty(n_out, Kp, dtype=self.act_dtype, device=dev)
        self._branch_norm(x, pend, gain["final.norm"], out=hf, ldo=Kp, gather=rows)
        raw = self._linear(hf, self._packed["head"], n_out)
        logits = torch.empty(n_out, V, dtype=torch.float32, device=dev)
        check(lib.evo_scale_logits(ptr(raw), self._packed["head"].Np, ptr(logits), n_out, V, cfg.logit_scale, self._dt, self._stream()), "evo_scale_logits")
        return logits
