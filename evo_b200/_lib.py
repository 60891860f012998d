"""ctypes binding of libevo_b200.so (the C ABI declared in include/evo_b200.h).

There is no CPU fallback and no other backend: if the shared library is missing or a
call fails, this module raises.  Build it with ``python -m evo_b200.build``."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libevo_b200.so")

EPI_NONE, EPI_BIAS, EPI_BIAS_RESID, EPI_RESID, EPI_GELU_GATE = range(5)
EPI_BIAS_ROPE = 6
EPI_HYENA_STEP = 7


class EvoError(RuntimeError):
    pass


class GemmParams(C.Structure):
    _fields_ = [("A", C.c_void_p), ("lda", C.c_int64), ("W", C.c_void_p), ("C", C.c_void_p), ("ldc", C.c_int64),
                ("bias", C.c_void_p), ("residual", C.c_void_p), ("ldr", C.c_int64),
                ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("epilogue", C.c_int), ("variant", C.c_int),
                ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("rope_L", C.c_int64), ("rope_cols", C.c_int64),
                ("c_peers", C.c_void_p), ("n_c_peers", C.c_int), ("peer_period", C.c_int64), ("peer_inner", C.c_int64), ("peer_row0", C.c_int64)]


class GemmSmallMParams(C.Structure):
    _fields_ = [("A", C.c_void_p), ("lda", C.c_int64), ("W", C.c_void_p), ("C", C.c_void_p), ("ldc", C.c_int64),
                ("bias", C.c_void_p), ("residual", C.c_void_p), ("ldr", C.c_int64),
                ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("epilogue", C.c_int),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("fir_state", C.c_void_p), ("state", C.c_void_p), ("fir_w", C.c_void_p), ("fir_b", C.c_void_p), ("Dskip", C.c_void_p),
                ("poles", C.c_void_p), ("residues", C.c_void_p)]


class HyenaParams(C.Structure):
    _fields_ = [("z", C.c_void_p), ("y", C.c_void_p), ("fir_w", C.c_void_p), ("fir_b", C.c_void_p), ("Dskip", C.c_void_p),
                ("poles", C.c_void_p), ("residues", C.c_void_p),
                ("B", C.c_int), ("L", C.c_int64), ("D", C.c_int), ("S", C.c_int), ("nheads", C.c_int),
                ("halo", C.c_void_p), ("state_in", C.c_void_p), ("state_out", C.c_void_p), ("fir_state_out", C.c_void_p),
                ("force_segments", C.c_int), ("state_only", C.c_int), ("reuse_segment_states", C.c_int)]


class AttnParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
                ("q_tok_stride", C.c_int64), ("kv_tok_stride", C.c_int64),
                ("q_batch_stride", C.c_int64), ("kv_batch_stride", C.c_int64),
                ("B", C.c_int), ("Lq", C.c_int64), ("Lk", C.c_int64), ("H", C.c_int), ("hd", C.c_int),
                ("q_pos0", C.c_int64), ("softmax_scale", C.c_float),
                ("out_peers", C.c_void_p), ("n_out_peers", C.c_int), ("out_rows_per_peer", C.c_int64), ("out_row_stride", C.c_int64), ("out_col0", C.c_int64)]


class ScoreParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("W", C.c_void_p), ("targets", C.c_void_p), ("logprobs", C.c_void_p), ("entropy", C.c_void_p),
                ("M", C.c_int64), ("V", C.c_int), ("K", C.c_int64), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class LoopParams(C.Structure):
    _fields_ = [("forced", C.c_void_p), ("n_forced", C.c_int64), ("forced_stride", C.c_int64),
                ("picked", C.c_void_p), ("picked_stride", C.c_int64),
                ("kept_logits", C.c_void_p), ("n_out", C.c_int64),
                ("top_k", C.c_int32), ("top_p", C.c_float), ("temperature", C.c_float),
                ("seed", C.c_uint64), ("step0", C.c_int64)]


class ResidNormParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("ldy", C.c_int64), ("y_dtype", C.c_int), ("y_scale", C.c_float),
                ("x_add", C.c_void_p), ("weight", C.c_void_p), ("weight_offset", C.c_float), ("eps", C.c_float),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("out_dtype", C.c_int),
                ("B", C.c_int), ("seq_len", C.c_int64), ("halo", C.c_int64), ("D", C.c_int),
                ("halo_src", C.c_void_p), ("gather", C.c_void_p)]


class CausalConvParams(C.Structure):
    _fields_ = [("inp", C.c_void_p), ("weight", C.c_void_p), ("out", C.c_void_p), ("ldo", C.c_int64), ("out_dtype", C.c_int),
                ("carry_out", C.c_void_p), ("B", C.c_int), ("seq_len", C.c_int64), ("D", C.c_int), ("taps", C.c_int)]


class Hgrn2Params(C.Structure):
    _fields_ = [("q", C.c_void_p), ("f", C.c_void_p), ("v", C.c_void_p), ("ld", C.c_int64),
                ("f_bias", C.c_void_p), ("lower", C.c_void_p), ("norm_w", C.c_void_p), ("eps", C.c_float),
                ("state", C.c_void_p), ("zero_start", C.c_int),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("dtype", C.c_int),
                ("B", C.c_int), ("L", C.c_int64), ("H", C.c_int), ("dk", C.c_int), ("dv", C.c_int)]


class WindowAttnParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_tok_stride", C.c_int64),
                ("k", C.c_void_p), ("v", C.c_void_p), ("k_tok_stride", C.c_int64), ("v_tok_stride", C.c_int64),
                ("k_batch_stride", C.c_int64), ("v_batch_stride", C.c_int64),
                ("gate", C.c_void_p), ("gate_tok_stride", C.c_int64),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("dtype", C.c_int),
                ("B", C.c_int), ("Lq", C.c_int64), ("H", C.c_int), ("G", C.c_int), ("dk", C.c_int), ("dv", C.c_int), ("n_maps", C.c_int),
                ("q_pos0", C.c_int64), ("pos_dev", C.c_void_p), ("window", C.c_int64), ("keep_first", C.c_int64),
                ("scale", C.c_float), ("lambda_", C.c_float), ("head_norm", C.c_int), ("norm_eps", C.c_float), ("out_scale", C.c_float), ("gate_per_head", C.c_int),
                ("softcap", C.c_float), ("sink", C.c_void_p), ("pool", C.c_int64), ("pool_k", C.c_void_p), ("pool_v", C.c_void_p),
                ("pool_tok_stride", C.c_int64), ("pool_batch_stride", C.c_int64), ("dist_r1", C.c_void_p), ("dist_r2", C.c_void_p)]


class BranchNormParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("ldy", C.c_int64),
                ("gate", C.c_void_p), ("ldg", C.c_int64), ("gate_bias", C.c_void_p),
                ("post_norm", C.c_int), ("post_gain", C.c_float), ("replace", C.c_int), ("row_add", C.c_void_p),
                ("gain", C.c_float), ("eps", C.c_float), ("out", C.c_void_p), ("ldo", C.c_int64),
                ("concat", C.c_int), ("cat", C.c_void_p), ("dtype", C.c_int), ("rows", C.c_int64), ("D", C.c_int), ("gather", C.c_void_p)]


class MinGruParams(C.Structure):
    _fields_ = [("z", C.c_void_p), ("u", C.c_void_p), ("g", C.c_void_p), ("ld", C.c_int64),
                ("z_bias", C.c_void_p), ("u_bias", C.c_void_p), ("state", C.c_void_p), ("zero_start", C.c_int),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("dtype", C.c_int), ("B", C.c_int), ("L", C.c_int64), ("W", C.c_int)]


class LatentPrepParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("ldq", C.c_int64), ("dkv", C.c_void_p), ("ld_dkv", C.c_int64),
                ("norm_w", C.c_void_p), ("eps", C.c_float), ("freq", C.c_void_p),
                ("cache", C.c_void_p), ("cache_row", C.c_int64), ("cache_batch_stride", C.c_int64), ("rank_pad", C.c_int),
                ("B", C.c_int), ("L", C.c_int64), ("H", C.c_int), ("dim", C.c_int), ("rot", C.c_int), ("rank", C.c_int),
                ("pos0", C.c_int64), ("pos_dev", C.c_void_p), ("dtype", C.c_int), ("rot_dims", C.c_int)]


class LatentDecodeParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("ldq", C.c_int64),
                ("cache", C.c_void_p), ("cache_row", C.c_int64), ("cache_batch_stride", C.c_int64), ("rank_pad", C.c_int),
                ("uk", C.c_void_p), ("uv", C.c_void_p), ("gate", C.c_void_p), ("ld_gate", C.c_int64),
                ("out", C.c_void_p), ("ldo", C.c_int64),
                ("B", C.c_int), ("Lq", C.c_int64), ("H", C.c_int), ("dim", C.c_int), ("rot", C.c_int), ("rank", C.c_int), ("vdim", C.c_int),
                ("pos0", C.c_int64), ("pos_dev", C.c_void_p), ("window", C.c_int64), ("scale", C.c_float), ("dtype", C.c_int), ("max_keys", C.c_int64)]


SUM_NORM_BRANCHES = 3


class SumNormParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p * SUM_NORM_BRANCHES), ("ldy", C.c_int64 * SUM_NORM_BRANCHES),
                ("norm_w", C.c_void_p * SUM_NORM_BRANCHES), ("scale", C.c_float * SUM_NORM_BRANCHES), ("n_branches", C.c_int),
                ("eps", C.c_float), ("out", C.c_void_p * 2), ("w", C.c_void_p * 2), ("ldo", C.c_int64),
                ("dtype", C.c_int), ("rows", C.c_int64), ("D", C.c_int), ("gather", C.c_void_p)]


class ConvActParams(C.Structure):
    _fields_ = [("inp", C.c_void_p), ("ld", C.c_int64), ("weight", C.c_void_p), ("bias", C.c_void_p),
                ("carry", C.c_void_p), ("zero_start", C.c_int), ("out", C.c_void_p), ("ldo", C.c_int64),
                ("B", C.c_int), ("L", C.c_int64), ("C", C.c_int), ("taps", C.c_int), ("act", C.c_int), ("dtype", C.c_int)]


class GatedDeltaParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("ld", C.c_int64),
                ("b", C.c_void_p), ("a", C.c_void_p), ("gate", C.c_void_p), ("ldz", C.c_int64),
                ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("norm_w", C.c_void_p),
                ("eps", C.c_float), ("unit_eps", C.c_float), ("q_scale", C.c_float),
                ("state", C.c_void_p), ("zero_start", C.c_int), ("out", C.c_void_p), ("ldo", C.c_int64), ("dtype", C.c_int),
                ("B", C.c_int), ("L", C.c_int64), ("H", C.c_int), ("G", C.c_int), ("dk", C.c_int), ("dv", C.c_int)]


class SsdParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("Bm", C.c_void_p), ("Cm", C.c_void_p), ("ld", C.c_int64), ("dt", C.c_void_p), ("ld_dt", C.c_int64),
                ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("D", C.c_void_p), ("state", C.c_void_p), ("zero_start", C.c_int),
                ("y", C.c_void_p), ("dtype", C.c_int), ("B", C.c_int), ("L", C.c_int64), ("H", C.c_int), ("G", C.c_int), ("N", C.c_int), ("dv", C.c_int)]


class QkPrepParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("ld", C.c_int64),
                ("q_bias", C.c_void_p), ("k_bias", C.c_void_p), ("v_bias", C.c_void_p),
                ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p), ("eps", C.c_float), ("freq", C.c_void_p), ("rot_dims", C.c_int),
                ("cache", C.c_void_p), ("cache_row", C.c_int64), ("cache_batch_stride", C.c_int64),
                ("B", C.c_int), ("L", C.c_int64), ("H", C.c_int), ("G", C.c_int), ("dk", C.c_int), ("dv", C.c_int),
                ("pos0", C.c_int64), ("pos_dev", C.c_void_p), ("dtype", C.c_int),
                ("norm_per_head", C.c_int), ("q_temp_coef", C.c_float), ("q_temp_every", C.c_int64)]


class MoeRouteParams(C.Structure):
    _fields_ = [("h", C.c_void_p), ("ldh", C.c_int64), ("router_w", C.c_void_p), ("correction", C.c_void_p),
                ("weights", C.c_void_p), ("ldw", C.c_int64), ("chosen", C.c_void_p),
                ("rows", C.c_int64), ("D", C.c_int), ("E", C.c_int), ("top", C.c_int), ("n_extra", C.c_int),
                ("score_fn", C.c_int), ("groups", C.c_int), ("keep", C.c_int), ("normalize", C.c_int), ("norm_eps", C.c_float), ("scale", C.c_float), ("dtype", C.c_int)]


class PostNormParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_in", C.c_void_p),
                ("y", C.c_void_p * 2), ("ldy", C.c_int64 * 2), ("scale", C.c_float * 2), ("n_in", C.c_int),
                ("norm_w", C.c_void_p), ("norm_b", C.c_void_p), ("eps", C.c_float),
                ("stack", C.c_void_p), ("stack_stride", C.c_int64), ("mix_n", C.c_int), ("mix_w", C.c_void_p),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("out_norm_w", C.c_void_p), ("out_norm_b", C.c_void_p),
                ("dtype", C.c_int), ("rows", C.c_int64), ("D", C.c_int), ("gather", C.c_void_p)]


class MlstmParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("ld", C.c_int64),
                ("gi", C.c_void_p), ("gf", C.c_void_p), ("ldg", C.c_int64),
                ("i_bias", C.c_void_p), ("f_bias", C.c_void_p), ("cap", C.c_float), ("q_scale", C.c_float), ("den_eps", C.c_float),
                ("gate", C.c_void_p), ("ld_gate", C.c_int64), ("norm_w", C.c_void_p), ("eps", C.c_float),
                ("state", C.c_void_p), ("mstate", C.c_void_p), ("zero_start", C.c_int),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("dtype", C.c_int),
                ("B", C.c_int), ("L", C.c_int64), ("H", C.c_int), ("dk", C.c_int), ("dv", C.c_int)]


# name -> (restype, argtypes); every symbol include/evo_b200.h declares
SIGNATURES = {
    "evo_last_error": (C.c_char_p, []),
    "evo_abi_version": (C.c_int, []),
    "evo_launch_count": (C.c_int64, []),
    "evo_reset_launch_count": (None, []),
    "evo_note_graph_replay": (None, [C.c_int64]),
    "evo_embed": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "evo_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_void_p]),
    "evo_gemm": (C.c_int, [C.POINTER(GemmParams), C.c_void_p]),
    "evo_gemm_smallm_workspace": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int]),
    "evo_gemm_smallm": (C.c_int, [C.POINTER(GemmSmallMParams), C.c_void_p]),
    "evo_set_pdl": (C.c_int, [C.c_int]),
    "evo_hyena_fwd_workspace": (C.c_size_t, [C.POINTER(HyenaParams)]),
    "evo_hyena_fwd": (C.c_int, [C.POINTER(HyenaParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_hyena_step": (C.c_int, [C.c_void_p] * 9 + [C.c_int] * 4 + [C.c_void_p]),
    "evo_hyena_combine_states": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "evo_peer_publish": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "evo_peer_wait": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "evo_rope_tables": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_float, C.c_void_p]),
    "evo_rotary_qk": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "evo_attn_fwd_workspace": (C.c_size_t, [C.POINTER(AttnParams), C.c_int]),
    "evo_attn_fwd_ws": (C.c_int, [C.POINTER(AttnParams), C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_kv_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_void_p]),
    "evo_gelu_gate_interleaved": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "evo_decode_qkv_prep": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_void_p]),
    "evo_decode_attn_workspace": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "evo_decode_attn": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_advance_position": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p]),
    "evo_sample": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_uint64, C.c_uint64, C.c_void_p]),
    "evo_sample_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "evo_advance_counters": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "evo_unembed_score_workspace": (C.c_size_t, [C.c_int64, C.c_int]),
    "evo_unembed_score": (C.c_int, [C.POINTER(ScoreParams), C.c_void_p]),
    "evo_tokenize_pad": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "evo_logprobs": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "evo_embed_f32": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "evo_resid_norm": (C.c_int, [C.POINTER(ResidNormParams), C.c_void_p]),
    "evo_causal_conv": (C.c_int, [C.POINTER(CausalConvParams), C.c_void_p]),
    "evo_polynorm": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "evo_softcap_logits": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "evo_copy_rows": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int64, C.c_int, C.c_int64, C.c_void_p, C.c_int, C.c_void_p]),
    "evo_hgrn2_workspace": (C.c_size_t, [C.POINTER(Hgrn2Params)]),
    "evo_hgrn2_fwd": (C.c_int, [C.POINTER(Hgrn2Params), C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_window_attn_fwd": (C.c_int, [C.POINTER(WindowAttnParams), C.c_void_p]),
    "evo_gemm_simt": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "evo_embed_pair_f32": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_float,
                                     C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "evo_branch_norm": (C.c_int, [C.POINTER(BranchNormParams), C.c_void_p]),
    "evo_glu_act": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "evo_scale_logits": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "evo_mingru_workspace": (C.c_size_t, [C.POINTER(MinGruParams)]),
    "evo_mingru_fwd": (C.c_int, [C.POINTER(MinGruParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_latent_prep": (C.c_int, [C.POINTER(LatentPrepParams), C.c_void_p]),
    "evo_latent_attn_decode_workspace": (C.c_size_t, [C.POINTER(LatentDecodeParams)]),
    "evo_latent_attn_decode": (C.c_int, [C.POINTER(LatentDecodeParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_moe_count": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "evo_moe_scatter": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "evo_gather_rows": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "evo_moe_combine": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "evo_sum_norm": (C.c_int, [C.POINTER(SumNormParams), C.c_void_p]),
    "evo_conv_act": (C.c_int, [C.POINTER(ConvActParams), C.c_void_p]),
    "evo_xielu": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "evo_gated_group_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "evo_gated_delta_workspace": (C.c_size_t, [C.POINTER(GatedDeltaParams)]),
    "evo_gated_delta_fwd": (C.c_int, [C.POINTER(GatedDeltaParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_ssd_fwd": (C.c_int, [C.POINTER(SsdParams), C.c_void_p]),
    "evo_qk_prep": (C.c_int, [C.POINTER(QkPrepParams), C.c_void_p]),
    "evo_pool_rows": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int64, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_void_p]),
    "evo_moe_route_ex": (C.c_int, [C.POINTER(MoeRouteParams), C.c_void_p]),
    "evo_post_norm": (C.c_int, [C.POINTER(PostNormParams), C.c_void_p]),
    "evo_mlstm_workspace": (C.c_size_t, [C.POINTER(MlstmParams)]),
    "evo_mlstm_fwd": (C.c_int, [C.POINTER(MlstmParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "evo_moe_route": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]),
}

_lib = None


def lib():
    """The loaded library (loads on first use; raises if it is not built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EvoError(f"{LIB_PATH} is missing: the CUDA extension is not built (run `python -m evo_b200.build`). "
                           "evo_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str = ""):
    if rc != 0:
        msg = lib().evo_last_error()
        raise EvoError(f"{what or 'evo_b200'} failed (rc={rc}): {msg.decode() if msg else ''}")


def ptr(t):
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else C.c_void_p(t.data_ptr())
