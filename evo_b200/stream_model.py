"""Shared base of the model families that keep the residual stream in fp32 and are described by a flat table of checkpoint
tensors (Zaverax, Movalorn, Nelovik): weight holding and strict loading, the padded GEMM weights, the linear-layer dispatch
(tcgen05 GEMMs for bf16 activations, the CUDA-core fp32 GEMM for the all-fp32 mode), the inference-state holders, the
forward protocol and the on-device generation loop.  A family provides `_ensure_packed()` and
`_body(ids, B, L, state, offset, pos_dev=None, rows=None) -> fp32 logits`; everything that drives a model -- the generation loop,
the scheduler, the trace replay, the command line -- talks to the methods defined here.

Protocol (the same as StripedHyena's):
    model(ids) -> (logits, None)                          stateless, whole sequences
    model(ids, inference_params_dict=d) -> (logits, d)    continues from the caches in d at d["mha"].seqlen_offset
    model.initialize_inference_params()                   the framework's two state holders
    model.decode_loop(...)                                one CUDA graph per generated token
State is keyed by RUN index (a looped layer has one entry per pass): d["mha"].key_value_memory_dict[r] for caches that grow
with the sequence, d["hyena"].state_dict[r] / fir_state_dict[r] for fixed-size recurrent state.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import torch
import torch.nn as nn

from . import _lib
from ._lib import EPI_NONE, ConvActParams, GatedDeltaParams, check, ptr
from .engine import KernelOps
from .stripedhyena.cache import InferenceParams, RecurrentInferenceParams


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class _Packed:
    """A linear layer's weight in the GEMMs' layout: (Np, Kp) bf16, zero rows / columns past (N, K)."""

    def __init__(self, w: torch.Tensor):
        self.N, self.K = w.shape
        self.Np, self.Kp = _round_up(self.N, 256), _round_up(self.K, 64)
        self.w = torch.zeros(self.Np, self.Kp, dtype=torch.bfloat16, device=w.device)
        self.w[:self.N, :self.K] = w.to(torch.bfloat16)


class StreamDecoder(KernelOps, nn.Module):
    architecture = None
    gemm_env = "EVO_B200_STREAM_GEMM"          # "simt": linear layers of the bf16 path on the CUDA-core GEMM (comparator)
    fir_taps = 0                               # taps of a short convolution whose carried rows live in the recurrent holder

    def __init__(self, config, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("activation dtype must be torch.bfloat16 or torch.float32")
        self.config = config
        self.act_dtype = dtype
        self.weights: Dict[str, torch.Tensor] = {}
        for name, shape in config.tensor_shapes().items():
            self.weights[name] = torch.zeros(shape, dtype=torch.bfloat16)
        self._packed = None
        # linear layers of the bf16 path: "tc" = tcgen05 GEMMs, "simt" = the CUDA-core GEMM (comparator)
        self.gemm_path = os.environ.get(self.gemm_env, "tc")
        self.gemm_variant = int(os.environ.get("EVO_B200_GEMM_VARIANT", "0"))
        self.gemm_variant_gate = self.gemm_variant
        self.decode_graph = os.environ.get("EVO_B200_DECODE_GRAPH", "1") != "0"
        self._smallm_ws = None
        self._decode = None
        self._loop = None
        self._prof = None
        self._tap = None          # set to a list: receives the fp32 stream after every run (bring-up / tests)

    # ---- parameters ----------------------------------------------------------------------------
    def state_dict(self, *a, **kw):
        return dict(self.weights)

    def load_state_dict(self, state_dict, strict: bool = True, **kw):
        missing = [k for k in self.weights if k not in state_dict]
        unexpected = [k for k in state_dict if k not in self.weights]
        errors = []
        for k, v in state_dict.items():
            if k in self.weights:
                if tuple(v.shape) != tuple(self.weights[k].shape):
                    errors.append(f"size mismatch for {k}: checkpoint {tuple(v.shape)}, model {tuple(self.weights[k].shape)}")
                else:
                    self.weights[k] = v.to(device=self.weights[k].device, dtype=torch.bfloat16).contiguous()
        if errors or (strict and (missing or unexpected)):
            raise RuntimeError(f"Error(s) in loading state_dict for {type(self).__name__}: missing {missing}, unexpected {unexpected}, {errors}")
        self._invalidate()
        return missing, unexpected

    def _invalidate(self):
        self._packed = None
        self._decode = None
        self._loop = None

    def _apply(self, fn, *a, **kw):
        out = super()._apply(fn, *a, **kw)
        for k, v in self.weights.items():
            moved = fn(v)
            self.weights[k] = moved if moved.dtype == torch.bfloat16 else moved.to(torch.bfloat16)      # .float() / .half() do not apply to the checkpoint's bf16
        self._invalidate()
        return out

    @property
    def device(self):
        return self.weights["embed"].device

    def eval(self):
        return self

    def _ensure_packed(self):
        raise NotImplementedError

    def _body(self, ids, B, L, ipd, off: int, pos_dev=None, rows=None):
        raise NotImplementedError

    # ---- state -----------------------------------------------------------------------------------
    def initialize_inference_params(self, max_seqlen: Optional[int] = None, max_batch_size: Optional[int] = None):
        return {
            "mha": InferenceParams(max_seqlen=max_seqlen or self.config.max_seqlen, max_batch_size=max_batch_size or self.config.max_batch_size, seqlen_offset=0),
            "hyena": RecurrentInferenceParams(fir_filter_length=self.fir_taps, state_dim=0, seqlen_offset=0),
        }

    def _kv_rows(self, ip: InferenceParams, r: int, width: int, B: int, off: int, L: int, pos_dev=None):
        """The cache of run r, (max_batch, max_seqlen, width) in the activation dtype, zero-filled: allocated on first use and
        doubled (outside a captured step) when rows [off, off + L) would not fit.  Rows are never overwritten or moved within a
        sequence, so a window only limits what the kernels read."""
        cache = ip.key_value_memory_dict.get(r)
        dev = self.device
        if cache is None:
            cache = ip.key_value_memory_dict[r] = torch.zeros(ip.max_batch_size, max(ip.max_seqlen, off + L), width, dtype=self.act_dtype, device=dev)
        if B > cache.shape[0]:
            raise _lib.EvoError(f"KV cache too small: batch {B} > {cache.shape[0]}")
        if off + L > cache.shape[1]:
            if pos_dev is not None:             # inside a captured step the cache cannot move
                raise _lib.EvoError(f"KV cache too small: length {off + L} > {cache.shape[1]}")
            grown = torch.zeros(cache.shape[0], max(off + L, 2 * cache.shape[1]), width, dtype=self.act_dtype, device=dev)
            grown[:, :off] = cache[:, :off]
            cache = ip.key_value_memory_dict[r] = grown
            ip.max_seqlen = max(ip.max_seqlen, cache.shape[1])
        return cache

    def _cache_tokens(self, key, cache) -> int:
        """Tokens of a sequence that the cache under `key` has room for (a family that keeps one row per several tokens overrides this)."""
        return cache.shape[1]

    # ---- kernels ---------------------------------------------------------------------------------
    @property
    def _dt(self) -> int:
        return 1 if self.act_dtype == torch.float32 else 0

    def _linear(self, a, pk: _Packed, M: int, out=None):
        """(M, Kp) activations -> (M, Np): rows of A are padded with zeros up to Kp by their producers.  out: rows of a (.., Np) buffer to fill."""
        if out is None:
            out = torch.empty(M, pk.Np, dtype=self.act_dtype, device=a.device)
        if self._dt or self.gemm_path == "simt":
            self._record(f"gemm_simt/{pk.N}x{pk.K}", 2.0 * M * pk.N * pk.K, lambda: check(_lib.lib().evo_gemm_simt(
                ptr(a), pk.Kp, ptr(pk.w), pk.Kp, ptr(out), pk.Np, M, pk.N, pk.K, self._dt, self._stream()), "evo_gemm_simt"))
        elif M <= 64:
            self._gemm_smallm(a, pk.w, out, M, pk.Np, pk.Kp, EPI_NONE)
        else:
            self._gemm(a, pk.w, out, M, pk.Np, pk.Kp, EPI_NONE, variant=2 if M <= 512 else self.gemm_variant)
        return out

    # ---- mixers shared by several families ---------------------------------------------------------
    def _conv(self, r, src_ptr, ld, weight, bias, channels, taps, B, L, rec, fresh):
        """SiLU(short convolution) of `channels` columns starting at src_ptr -> (B*L, channels); the carried inputs live in rec.fir_state_dict[r]."""
        dev = weight.device
        out = torch.empty(B * L, channels, dtype=self.act_dtype, device=dev)
        carry, zero = None, 1
        if taps > 1:
            carry = rec.fir_state_dict.get(r)
            zero = 0
            if carry is None or fresh:
                if carry is None:
                    carry = rec.fir_state_dict[r] = torch.empty(B, taps - 1, channels, dtype=torch.float32, device=dev)
                zero = 1
        cp = ConvActParams(inp=src_ptr, ld=ld, weight=weight.data_ptr(), bias=bias.data_ptr() if bias is not None else None,
                           carry=carry.data_ptr() if carry is not None else None, zero_start=zero, out=out.data_ptr(), ldo=channels,
                           B=B, L=L, C=channels, taps=taps, act=1, dtype=self._dt)
        self._record("conv_act", 2.0 * out.element_size() * B * L * channels, lambda: check(_lib.lib().evo_conv_act(C.byref(cp), self._stream()), "evo_conv_act"))
        return out

    def _matrix_state(self, r, rec, B, H, dk, dv, fresh):
        state = rec.state_dict.get(r)
        if state is None:
            state = rec.state_dict[r] = torch.empty(B, H, dk, dv, dtype=torch.float32, device=self.device)
            return state, 1
        return state, 1 if fresh else 0

    def _delta_mixer(self, r, i, m, h, B, L, rec, fresh):
        """Gated delta rule of layer i (tensors l<i>.mix.*; m: heads, kv_heads, dim, vdim, taps) on h (M, Kp) -> (output projection, its row stride)."""
        pk = self._packed["layers"][i]
        M, dev = B * L, h.device
        w = self.weights
        z = self._linear(h, pk["in"], M)
        esz, ldz = z.element_size(), pk["in"].Np
        qk, vw = m.kv_heads * m.dim, m.heads * m.vdim
        cw = 2 * qk + vw
        c = self._conv(r, z.data_ptr(), ldz, pk["conv"], None, cw, m.taps, B, L, rec, fresh)
        state, zero = self._matrix_state(r, rec, B, m.heads, m.dim, m.vdim, fresh)
        ldo = _round_up(vw, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        p = f"l{i}.mix."
        gp = GatedDeltaParams(q=c.data_ptr(), k=c.data_ptr() + qk * esz, v=c.data_ptr() + 2 * qk * esz, ld=cw,
                              b=z.data_ptr() + (cw + vw) * esz, a=z.data_ptr() + (cw + vw + m.heads) * esz, gate=z.data_ptr() + cw * esz, ldz=ldz,
                              A_log=w[p + "A_log"].data_ptr(), dt_bias=w[p + "dt_bias"].data_ptr(), norm_w=w[p + "norm"].data_ptr(),
                              eps=self.config.eps, unit_eps=1e-6, q_scale=m.dim ** -0.5, state=state.data_ptr(), zero_start=zero,
                              out=out.data_ptr(), ldo=ldo, dtype=self._dt, B=B, L=L, H=m.heads, G=m.kv_heads, dk=m.dim, dv=m.vdim)
        nws = _lib.lib().evo_gated_delta_workspace(C.byref(gp))
        ws = torch.empty(nws, dtype=torch.uint8, device=dev) if nws else None
        self._record("gated_delta", 4.0 * M * m.heads * m.dim * m.vdim, lambda: check(_lib.lib().evo_gated_delta_fwd(C.byref(gp), ptr(ws), nws, self._stream()), "evo_gated_delta_fwd"))
        return self._linear(out, pk["out"], M), pk["out"].Np

    def _run_chosen_experts(self, h, M, chosen, experts, ff, E, top):
        """Only the chosen experts of a mixture: the (token, choice) pairs of `chosen` (M, top) int32 are sorted by expert, and every
        expert ([gate ; up] and down weights, packed, hidden size ff, SiLU-gated) runs on its slice of the gathered rows of h (M, Kp).
        Returns (ys, slot_of): the experts' outputs in sorted order and the slot of every pair, for evo_moe_combine.  The per-expert
        row counts come back to the host (one round trip), so this does not run inside a captured step."""
        dev, lib = h.device, _lib.lib()
        n, esz = M * top, h.element_size()
        counts = torch.zeros(2, E, dtype=torch.int32, device=dev)                      # row 0: counts, row 1: the scatter's cursors
        check(lib.evo_moe_count(ptr(chosen), n, E, ptr(counts), self._stream()), "evo_moe_count")
        cnt = counts[0].cpu()                                                           # the one host round trip of the layer
        off = torch.zeros(E + 1, dtype=torch.int64)
        off[1:] = torch.cumsum(cnt.to(torch.int64), 0)
        offsets = off[:E].to(torch.int32).to(dev)
        total = int(off[E])
        perm = torch.empty(max(total, 1), dtype=torch.int32, device=dev)
        slot_of = torch.empty(M, top, dtype=torch.int32, device=dev)
        check(lib.evo_moe_scatter(ptr(chosen), n, top, E, ptr(offsets), C.c_void_p(counts.data_ptr() + 4 * E), ptr(perm), ptr(slot_of), self._stream()), "evo_moe_scatter")
        Kp = h.shape[1]
        hs = torch.empty(max(total, 1), Kp, dtype=self.act_dtype, device=dev)
        self._record("moe_gather", 2.0 * total * Kp * esz, lambda: check(lib.evo_gather_rows(ptr(h), Kp * esz, ptr(hs), Kp * esz, ptr(perm), total, Kp * esz, self._stream()), "evo_gather_rows"))
        down0 = experts[0][1]
        ys = torch.empty(max(total, 1), down0.Np, dtype=self.act_dtype, device=dev)
        for e in range(E):
            lo, ne = int(off[e]), int(cnt[e])
            if ne == 0:
                continue
            up, down = experts[e]
            z = self._linear(hs[lo:lo + ne], up, ne)
            a = torch.empty(ne, down.Kp, dtype=self.act_dtype, device=dev)
            self._record("glu_act", 3.0 * esz * ne * ff, lambda: check(lib.evo_glu_act(
                ptr(z), C.c_void_p(z.data_ptr() + ff * esz), up.Np, ptr(a), down.Kp, ne, ff, 1, None, 0, 0, 0, 0, self._dt, self._stream()), "evo_glu_act"))
            self._linear(a, down, ne, out=ys[lo:lo + ne])
        return ys, slot_of

    # ---- forward ---------------------------------------------------------------------------------
    def forward(self, x, inference_params_dict=None, padding_mask=None, logits_rows=None):
        """ids (B, L) -> (fp32 logits (B, L, V), state).  With a state dict the call continues every sequence at
        state["mha"].seqlen_offset (the caller advances it, as the framework's generation loop does).
        logits_rows: flat indices into the (B*L) rows whose logits are wanted -> logits (len, V)."""
        if padding_mask is not None:
            raise NotImplementedError("padding_mask is not supported")
        if x.dim() != 2 or x.dtype not in (torch.int32, torch.int64):
            raise TypeError("input ids must be (batch, length) int32/int64")
        self._ensure_packed()
        dev = self.device
        if x.device != dev:
            raise _lib.EvoError(f"input ids on {x.device}, model on {dev}")
        x = x.contiguous()
        B, L = x.shape
        off = int(inference_params_dict["mha"].seqlen_offset) if inference_params_dict is not None else 0
        with torch.cuda.device(dev), torch.no_grad():
            rows = None
            if logits_rows is not None:
                rows = torch.as_tensor(logits_rows, dtype=torch.int64, device=dev).contiguous()
            logits = self._body(x, B, L, inference_params_dict, off, rows=rows)
        if rows is not None:
            return logits, inference_params_dict
        return logits.view(B, L, -1), inference_params_dict

    # ---- on-device generation loop: the whole step + token pick as one CUDA graph ------------------
    def decode_loop(self, first_token, ipd, n_steps, start_pos, *, top_k=1, top_p=0.0, temperature=1.0, forced=None, n_out=None, seed=None):
        """`n_steps` single-token steps without returning to the host: same contract as StripedHyena.decode_loop
        (step i feeds the token of step i-1; forced[:, i] while i < forced.shape[1], then picked on the device)."""
        lib = _lib.lib()
        dev = self.device
        x = first_token.reshape(-1, 1).contiguous()
        B, V = x.shape[0], self.config.vocab_size
        if V > 1024:
            raise _lib.EvoError("the device sampler handles vocabularies up to 1024; use the per-token host loop")
        mha_ip, rec = ipd["mha"], ipd["hyena"]
        n_forced = 0 if forced is None else int(forced.shape[1])
        n_out = n_steps - n_forced if n_out is None else n_out
        if n_out < 0:
            raise ValueError("more forced tokens than steps")
        for k, c in mha_ip.key_value_memory_dict.items():
            if start_pos + n_steps > self._cache_tokens(k, c):
                raise _lib.EvoError(f"sequence length {start_pos + n_steps} exceeds the KV cache ({self._cache_tokens(k, c)})")
        with torch.cuda.device(dev), torch.no_grad():
            self._ensure_packed()
            picked = torch.empty(B, max(n_out, 1), dtype=torch.long, device=dev)
            kept = torch.empty(B, max(n_out, 1), V, dtype=torch.float32, device=dev)
            forced_c = forced.to(dev, torch.long).contiguous() if n_forced else None
            if seed is None:
                seed = int(torch.randint(0, 2 ** 62, (1,)).item())
            lp = _lib.LoopParams(forced=forced_c.data_ptr() if n_forced else None, n_forced=n_forced, forced_stride=n_forced,
                                 picked=picked.data_ptr(), picked_stride=picked.shape[1], kept_logits=kept.data_ptr(), n_out=n_out,
                                 top_k=int(top_k), top_p=float(top_p), temperature=float(temperature), seed=seed, step0=0)
            key = ("loop", B, tuple((k, t.data_ptr()) for k, t in sorted(rec.state_dict.items())),
                   tuple((k, t.data_ptr()) for k, t in sorted(rec.fir_state_dict.items())),
                   tuple((k, t.data_ptr(), t.shape[1]) for k, t in sorted(mha_ip.key_value_memory_dict.items())))
            st = self._loop
            if st is None or st["key"] != key:
                st = {"key": key, "graph": None, "x": torch.empty(B, 1, dtype=torch.long, device=dev), "pos": torch.zeros(1, dtype=torch.int64, device=dev),
                      "step": torch.zeros(1, dtype=torch.int64, device=dev), "lp": torch.zeros(C.sizeof(_lib.LoopParams), dtype=torch.uint8, device=dev)}
                self._loop = st
            host = torch.frombuffer(bytearray(bytes(lp)), dtype=torch.uint8)
            st["lp"].copy_(host)
            st["pos"].fill_(int(start_pos))
            st["step"].zero_()
            st["x"].copy_(x.to(torch.long))

            def one_step():
                logits = self._body(st["x"], B, 1, ipd, 0, pos_dev=st["pos"])
                l16 = logits.to(torch.bfloat16)
                check(lib.evo_sample_step(ptr(l16), ptr(st["x"]), B, V, ptr(st["lp"]), ptr(st["step"]), self._stream()), "evo_sample_step")
                check(lib.evo_advance_counters(ptr(st["pos"]), ptr(st["step"]), 1, self._stream()), "evo_advance_counters")

            done = 0
            if st["graph"] is None or st.get("ws") != (self._smallm_ws.data_ptr() if self._smallm_ws is not None else 0):
                one_step()                      # eager step: allocates the workspaces the capture must not
                done = 1
                st["graph"] = None
                if self.decode_graph and n_steps > 1:
                    g = torch.cuda.CUDAGraph()
                    torch.cuda.synchronize()
                    n0 = lib.evo_launch_count()
                    with torch.cuda.graph(g):
                        one_step()
                    st["graph"], st["launches"] = g, lib.evo_launch_count() - n0
                    st["ws"] = self._smallm_ws.data_ptr() if self._smallm_ws is not None else 0
                    lib.evo_note_graph_replay(-st["launches"])
            for _ in range(done, n_steps):
                if st["graph"] is not None:
                    st["graph"].replay()
                    lib.evo_note_graph_replay(st["launches"])
                else:
                    one_step()
            mha_ip.seqlen_offset = rec.seqlen_offset = int(start_pos) + n_steps - 1
            return picked[:, :n_out], kept[:, :n_out]
