/* evo_b200 — C ABI of the B200-native StripedHyena forward engine.
 *
 * The reference (evo-design/evo) has no FFI: its boundary is the Python duck-type
 * of stripedhyena.model.StripedHyena (evo/models.py:141-150, evo/scoring.py:81,
 * evo/generation.py:117,152).  Everything that object computes is executed by the
 * entry points below; evo_b200/stripedhyena/model.py binds them with ctypes and
 * mirrors the Python protocol on top.  Each entry point cites the reference
 * operation it replaces (names inside stripedhyena==0.2.2 / flash_attn, which the
 * reference pins in requirements.txt:1 and README.md:47-48).
 *
 * Conventions
 *   - every pointer is a raw DEVICE pointer owned by the caller (a torch tensor);
 *     the library never allocates device memory except one small per-device cache
 *     (the SM -> die table and claim words of the GEMM's die-aware tile walk, csrc/die_map.cu);
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it;
 *   - bf16 tensors are row-major with the innermost dimension contiguous;
 *   - return value 0 = ok, negative = error; evo_last_error() has the message;
 *   - no exceptions cross the boundary, no torch types appear in signatures.
 */
#ifndef EVO_B200_H
#define EVO_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* evo_last_error(void);
int evo_abi_version(void);
/* #launches of evo_b200 kernels since the last evo_reset_launch_count() (bench: gpu_launches) */
int64_t evo_launch_count(void);
void evo_reset_launch_count(void);
/* a CUDA-graph replay launches the kernels captured in it without passing through this library: the host adds the
 * number of launches recorded at capture time, once per replay (and subtracts the ones counted while capturing,
 * when nothing ran), so that evo_launch_count() stays truthful */
void evo_note_graph_replay(int64_t launches);

/* ---- embedding gather: VocabParallelEmbedding.embed (evo/models.py:136 pins the key) ----
 * ids: int32 or int64 (ids_are_i64), n tokens; table (vocab, D) bf16; out (n, D) bf16. */
int evo_embed(const void* ids, int ids_are_i64, const void* table, void* out,
              int64_t n_tokens, int D, int vocab, void* stream);

/* ---- RMSNorm, non-flash branch of stripedhyena layers.RMSNorm.forward:
 * y = scale * x / (||x||_2 * D^-1/2 + eps), every intermediate rounded to bf16 as the
 * reference's bf16 tensor ops do.  x,out (rows, D) bf16; scale (D) bf16. */
int evo_rmsnorm(const void* x, const void* scale, void* out, int64_t rows, int D, float eps, void* stream);

/* ---- tensor-core linear layers (nn.Linear / ParallelGatedMLP / unembed) ----
 * C[M,N] = epilogue(A[M,K] . W[N,K]^T), bf16 in, fp32 accumulate (tcgen05, TMEM), bf16 out.
 * Requirements: K % 64 == 0, N % 256 == 0 (weights are re-packed once at load time,
 * see evo_b200/stripedhyena/model.py), lda/ldc/ldr in elements. */
enum {
  EVO_EPI_NONE = 0,       /* C = bf16(acc)                                              */
  EVO_EPI_BIAS = 1,       /* C = bf16(acc + bias[n])                nn.Linear(bias=True) */
  EVO_EPI_BIAS_RESID = 2, /* C = bf16(bf16(acc + bias[n]) + R[m,n]) out_filter_dense(z)+u, out_proj(ctx)+u */
  EVO_EPI_RESID = 3,      /* C = bf16(bf16(acc) + R[m,n])           l3(...) + u           */
  EVO_EPI_GELU_GATE = 4,  /* W rows interleaved in 128-row groups [l1 | l2]; C[M,N/2] =
                             bf16(gelu(bf16(acc1)) * bf16(acc2))    act(l1 x) * l2 x      */
  EVO_EPI_HYENA_STEP = 7, /* evo_gemm_smallm only: the Hyena in-projection (N = 3D, bias) with the decode step of the operator
                             (engine.step_fir + step_iir == evo_hyena_step) applied in the epilogue: a tile is one head's
                             [x2 | x1 | v] rows, C is y (M, D); fir_state / state are updated in place; z is never stored */
  EVO_EPI_BIAS_ROPE = 6   /* Wqkv projection with the rotary embedding applied where flash_attn applies it
                             (MHA.forward, mha.py:635-648): x = bf16(acc + bias[n]); columns n < rope_cols (q and k,
                             heads of 128) are rotated NeoX-style with the cos/sin row of the token's position
                             (row m -> table row m % rope_L; the caller offsets the tables by the first position),
                             fp32 arithmetic, one rounding on store -- evo_rotary_qk's result without a second pass */
};
typedef struct {
  const void* A; int64_t lda;
  const void* W;                 /* (N, K) row-major */
  void* C; int64_t ldc;
  const void* bias;              /* (N) bf16 or NULL */
  const void* residual; int64_t ldr;
  int64_t M, N, K;
  int epilogue;
  int variant;                   /* 0 = 2-CTA 256x256 tiles; 1 = 1-CTA 128x256 tiles; 2 = 1-CTA 128x64 weight-streaming tiles (small M);
                                    3 = like 2 with W given tile-major: (N/64, K/64, 64, 64), i.e. W.view(N/64,64,K/64,64).permute(0,2,1,3) */
  const void* rope_cos; const void* rope_sin;   /* EVO_EPI_BIAS_ROPE: (positions, 64) bf16 tables (evo_rope_tables) */
  int64_t rope_L;                /* tokens per sequence: row m uses table row m % rope_L */
  int64_t rope_cols;             /* columns [0, rope_cols) are rotated (2*H*128 for a qkv projection), the rest only get the bias */
  /* Peer-scattered output (n_c_peers > 0): the epilogue stores straight into up to 8 peer-mapped buffers over NVLink, i.e.
   * the Ulysses head<->sequence all-to-all of a sequence-parallel attention layer fused into the Wqkv GEMM (no NCCL, no
   * permute): column n of row m goes to c_peers[(n % peer_period) / peer_inner], element
   * (peer_row0 + m) * ldc + (n / peer_period) * peer_inner + n % peer_inner.  For qkv (3, H, 128) and P ranks:
   * peer_period = H*128, peer_inner = H/P*128, ldc = 3*peer_inner, peer_row0 = rank * rows.  C is ignored. */
  void* const* c_peers;          /* HOST array of n_c_peers device pointers */
  int n_c_peers; int64_t peer_period, peer_inner, peer_row0;
} evo_gemm_params;
int evo_gemm(const evo_gemm_params* p, void* stream);
/* Decode-step linear layer (M <= 64 rows): the same C = epilogue(A . W^T) with the same rounding points, as a
 * weight-streaming kernel (csrc/gemm_smallm.cu): swap-AB tcgen05 tiles (128 W rows x M), stream-K over all SMs,
 * deterministic fix-up through `workspace`, weight prefetch ahead of the programmatic-dependent-launch wait.
 * EVO_EPI_GELU_GATE is fused here (C is (M, N/2)); replaces ParallelGatedMLP / nn.Linear at L == 1
 * (evo/generation.py:152 step path).  workspace: evo_gemm_smallm_workspace() bytes, zero-filled ONCE by the caller
 * (the per-tile counters in it reset themselves); one workspace may serve every call on a stream. */
typedef struct {
  const void* A; int64_t lda;
  const void* W;                 /* (N, K) row-major; GELU_GATE: rows interleaved [l1 | l2] per 256 */
  void* C; int64_t ldc;
  const void* bias;
  const void* residual; int64_t ldr;
  int64_t M, N, K;               /* M <= 64, N % 256 == 0, K % 64 == 0 */
  int epilogue;                  /* EVO_EPI_* */
  void* workspace; size_t workspace_bytes;
  /* EVO_EPI_HYENA_STEP only (same tensors as evo_hyena_step): */
  void* fir_state; float* state;                 /* (M, 3D, 2) bf16, (M, D, 8, 2) fp32: in/out */
  const void* fir_w; const void* fir_b; const void* Dskip;
  const float* poles; const float* residues;
} evo_gemm_smallm_params;
size_t evo_gemm_smallm_workspace(int64_t M, int64_t N, int64_t K, int epilogue);
int evo_gemm_smallm(const evo_gemm_smallm_params* p, void* stream);
/* Programmatic dependent launch for the decode step.  0 = off (default); 1 = every decode-step kernel is launched with
 * programmatic stream serialization; 2 = only evo_gemm_smallm is (its weight prefetch then overlaps the small kernel or
 * the GEMM tail in front of it); 3 = evo_gemm_smallm and the few-row evo_rmsnorm; 4 = those and
 * evo_hyena_step (which fetches its filter parameters and states ahead of the wait).  Every decode-step kernel begins with griddepcontrol.launch_dependents and waits
 * (griddepcontrol.wait) before it first touches dependent data.  Process-wide switch; returns the previous value. */
int evo_set_pdl(int level);

/* ---- fused Hyena operator: HyenaInferenceEngine.parallel_fir + ParallelHyenaFilter.
 * compute_filter + parallel_iir (+ prefill_via_modal_fft) of stripedhyena 0.2.2, as one
 * modal scan.  z (B, L, 3D) bf16 -> y (B, L, D) bf16.
 *   fir_w (3D, 3) bf16 taps [t-2, t-1, t]; fir_b (3D) bf16; Dskip (D) bf16;
 *   poles, residues (D, S, 2) fp32 (re, im), S == 8; nheads: column-split head count.
 * Optional (NULL to skip):
 *   halo (B, 2, 3D) bf16: the two z rows preceding row 0 (sequence-sharded rank > 0, or
 *        a continued prefill); zero history otherwise.
 *   state_in (B, D, S, 2) fp32: modal state entering row 0.
 *   state_out (B, D, S, 2) fp32: modal state after the last row (== inference_params.
 *        state_dict[layer] of the reference, complex64).
 *   fir_state_out (B, 3D, 2) bf16: last two z rows (== fir_state_dict[layer]).
 * workspace: evo_hyena_fwd_workspace() bytes (segment carries when L is split). */
typedef struct {
  const void* z; void* y;
  const void* fir_w; const void* fir_b; const void* Dskip;
  const float* poles; const float* residues;
  int B; int64_t L; int D; int S; int nheads;
  const void* halo; const float* state_in;
  float* state_out; void* fir_state_out;
  int force_segments;            /* 0 = auto; >0 forces the number of L segments (tests) */
  int state_only;                /* 1 = compute state_out only (sequence-parallel carry pass); y may be NULL */
  int reuse_segment_states;      /* 1 = workspace already holds the zero-start segment end states of a preceding
                                    state_only call on the same z / halo / geometry: skip recomputing them */
} evo_hyena_params;
size_t evo_hyena_fwd_workspace(const evo_hyena_params* p);
int evo_hyena_fwd(const evo_hyena_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* decode step: engine.step_fir + step_iir.  u (B, 3D) bf16 -> y (B, D) bf16;
 * fir_state (B, 3D, 2) bf16 and state (B, D, S, 2) fp32 are updated in place. */
int evo_hyena_step(const void* u, void* y, void* fir_state, float* state,
                   const void* fir_w, const void* fir_b, const void* Dskip,
                   const float* poles, const float* residues,
                   int B, int D, int S, int nheads, void* stream);

/* combine per-rank end states into the state entering rank `rank`'s shard:
 * S_in = sum_{q<rank} p^{(rank-1-q)*seg_len} * ends[q].  ends (nranks, B, D, S, 2) fp32. */
int evo_hyena_combine_states(const float* ends, float* state_in, const float* poles,
                             int rank, int nranks, int64_t seg_len, int B, int D, int S, void* stream);

/* ---- peer-memory exchange for the sequence-parallel Hyena carry (NVLink stores + flags, no collective):
 * evo_peer_publish copies `bytes` from src into slot `rank` (slot_stride_bytes apart) of each peer buffer
 * peer_dsts[first_peer..last_peer] (device array of peer-mapped pointers) and then sets peer_flags[p][rank] = epoch
 * with system-scope release; evo_peer_wait blocks the stream until flags[first..last] >= epoch (acquire).
 * block_counter: one zero-initialised int of scratch on the calling device. */
int evo_peer_publish(const void* src, int64_t bytes, void* const* peer_dsts, int* const* peer_flags, int64_t slot_stride_bytes,
                     int rank, int first_peer, int last_peer, int epoch, int* block_counter, void* stream);
int evo_peer_wait(const int* flags, int first, int last, int epoch, void* stream);

/* ---- rotary tables + application (flash_attn layers/rotary.py:382-416,
 * ops/triton/rotary.py; stripedhyena LinearlyScaledRotaryEmbedding for 131k) ----
 * cos/sin (n_pos, hd/2) bf16 for positions pos0 .. pos0+n_pos-1, angle = (pos/scaling) * inv_freq[i]. */
int evo_rope_tables(void* cos_out, void* sin_out, const float* inv_freq, int64_t pos0, int64_t n_pos,
                    int half_dim, float scaling_factor, void* stream);
/* in-place NeoX rotary on q and k of qkv (B, L, 3, H, 128) bf16; cos/sin rows index the
 * position of row l directly (caller offsets the table for decode). */
int evo_rotary_qk(void* qkv, const void* cos, const void* sin, int B, int64_t L, int H, int hd, void* stream);

/* ---- causal attention core: flash_attn_qkvpacked_func (mha.py:122) ----
 * q: (B, Lq, H, 128) with row stride q_stride elements between tokens; k, v likewise over Lk
 * keys; query i attends keys j <= q_pos0 + i.  out (B, Lq, H*128) bf16 contiguous. */
typedef struct {
  const void* q; const void* k; const void* v; void* out;
  int64_t q_tok_stride, kv_tok_stride;     /* elements between consecutive tokens */
  int64_t q_batch_stride, kv_batch_stride; /* elements between batches */
  int B; int64_t Lq, Lk; int H; int hd;
  int64_t q_pos0;
  float softmax_scale;
  /* Peer-scattered output (n_out_peers > 0; variant 2, B == 1): query row i is stored into
   * out_peers[i / out_rows_per_peer] at element (i % out_rows_per_peer) * out_row_stride + out_col0 + h*128 -- the return
   * all-to-all of a sequence-parallel attention layer fused into the attention epilogue.  `out` is ignored. */
  void* const* out_peers;        /* HOST array of device pointers */
  int n_out_peers; int64_t out_rows_per_peer, out_row_stride, out_col0;
} evo_attn_params;
/* variant 0: V is transposed into the workspace first and consumed as a K-major operand;
 * variant 1: V is consumed in place as an MN-major operand (no workspace);
 * variant 2: ping-pong kernel: two query tiles per CTA, P kept in TMEM (A operand from TMEM), V in place;
 * variant 3: variant 2 with packed softmax arithmetic and 3 of every 8 exponentials evaluated on the FMA pipe (cubic). */
size_t evo_attn_fwd_workspace(const evo_attn_params* p, int variant);
int evo_attn_fwd_ws(const evo_attn_params* p, int variant, void* workspace, size_t workspace_bytes, void* stream);

/* append k,v of qkv (B, L, 3, H, hd) at rows [pos0, pos0+L) of the KV cache
 * (max_B, max_seqlen, 2, H, hd) bf16 — MHA._update_kv_cache (mha.py:344-370). */
int evo_kv_append(const void* qkv, void* cache, int B, int64_t L, int H, int hd,
                  int64_t pos0, int64_t max_seqlen, void* stream);

/* ---- decode step (L == 1), CUDA-graph friendly: the sequence position is read from DEVICE memory ----
 * evo_gelu_gate_interleaved: out[m, g*128+c] = bf16(gelu(t[m, g*256+c])) * t[m, g*256+128+c]; t (M, 2*ipad) is the
 *   plain GEMM output against the [l1 | l2]-interleaved weights (small-M tiles have no fused gate epilogue).
 * evo_decode_qkv_prep: rotary on q,k of qkv (B, 3, H, 128) at position *pos and append of k,v at cache row *pos
 *   (flash_attn_with_kvcache's rotary + cache-append half, mha.py:502-540).
 * evo_decode_attn: one query per sequence over cache keys [0, *pos] (the attention half); split-K over nsplit.
 * evo_advance_position: *pos += delta on the stream. */
int evo_gelu_gate_interleaved(const void* t, void* out, int64_t M, int ipad, void* stream);
int evo_decode_qkv_prep(void* qkv, void* cache, const void* cos, const void* sin, const int64_t* pos,
                        int B, int H, int hd, int64_t max_seqlen, void* stream);
size_t evo_decode_attn_workspace(int B, int H, int nsplit);
int evo_decode_attn(const void* qkv, const void* cache, void* out, const int64_t* pos, int B, int H, int hd,
                    int64_t max_seqlen, int nsplit, float softmax_scale, void* workspace, size_t workspace_bytes, void* stream);
int evo_advance_position(int64_t* pos, int64_t delta, void* stream);

/* ---- device-side sampler and generation loop: stripedhyena.sample.sample (evo/generation.py:162-167) and the host half
 * of the token loop (evo/generation.py:131-189) ----
 * evo_sample: logits (B, V) bf16 -> out (B) int64.  top_k == 1: argmax (first maximum); otherwise top-k (top_k <= 0:
 *   whole vocabulary) -> / temperature (bf16-rounded like the reference's tensor op) -> top-p tail mask (entries whose
 *   cumulative mass counted from the smallest up is <= 1 - top_p) -> multinomial.  Randomness: Philox4x32-10 keyed by
 *   (seed, step, row) -- reproducible, independent of launch order, CUDA-graph friendly.  V <= 1024.
 * evo_sample_step: the same inside the on-device loop.  Step index i = *step_dev (device); while i < n_forced the
 *   token is forced[row, i] (teacher-forced prompt tail), afterwards it is sampled with RNG step step0 + i and recorded:
 *   picked[row, i - n_forced] = token, kept_logits[row, i - n_forced, :] = float(logits[row]).  The token is also
 *   written to x[row], the next step's input.  All of evo_loop_params lives in DEVICE memory, so one captured graph
 *   serves every generate() call.
 * evo_advance_counters: *a += delta, *b += delta (either may be NULL). */
typedef struct {
  const int64_t* forced; int64_t n_forced; int64_t forced_stride;   /* (B, n_forced) int64 */
  int64_t* picked; int64_t picked_stride;                          /* (B, n_out) int64 or NULL */
  float* kept_logits; int64_t n_out;                               /* (B, n_out, V) fp32 or NULL */
  int32_t top_k; float top_p; float temperature;
  uint64_t seed; int64_t step0;
} evo_loop_params;
int evo_sample(const void* logits, int64_t* out, int B, int V, int top_k, float top_p, float temperature,
               uint64_t seed, uint64_t step, void* stream);
int evo_sample_step(const void* logits, int64_t* x, int B, int V, const evo_loop_params* loop_params_dev,
                    const int64_t* step_dev, void* stream);
int evo_advance_counters(int64_t* a, int64_t* b, int64_t delta, void* stream);

/* (test comparators -- cuBLASLt GEMM, CUDA-core attention, bf16 add -- live in tests/support/libevo_b200_test.so,
 *  not in this library) */

/* ---- scoring epilogue: evo/scoring.py:36-59 logits_to_logprobs ----
 * logits (rows, V) bf16; targets (rows) int64 (-1 = skip -> 0); out (rows) fp32 =
 * log_softmax(logits)[target], fp32 statistics. */
int evo_logprobs(const void* logits, const int64_t* targets, float* out, int64_t rows, int V, void* stream);


/* ---- batch front-end: evo/scoring.py:9-33 prepare_batch on the device ----
 * bytes: the sequences' raw bytes back to back (uint8, device); offsets (B+1) int64 (device): sequence b is
 * bytes[offsets[b] : offsets[b+1]].  ids_out (B, width) int32/int64 = [bos_id if prepend_bos] + bytes + pad_id ...
 * (CharLevelTokenizer.tokenize is the identity on bytes, evo/tokenizer.py:41).  width >= prepend_bos + max length. */
int evo_tokenize_pad(const void* bytes, const int64_t* offsets, void* ids_out, int ids_are_i64, int B, int64_t width,
                     int prepend_bos, int bos_id, int pad_id, void* stream);

/* ---- fused scoring head: unembed (tied embedding, N = vocab) + log_softmax + gather + entropy in one pass; the
 * (rows, V) logits never reach HBM (evo/scoring.py:36-59 logits_to_logprobs, :119-121 positional_entropies).
 * x (M, K) bf16 = final-norm output; W (V, K) bf16; targets (M) int64 (-1 = none -> logprob 0) or NULL.
 * logprobs[r] = bf16(x_r . W_t) - logsumexp_v(bf16(x_r . W_v)) in fp32 -- the logits are rounded to bf16 exactly where
 * the reference's logits tensor is, the statistics are fp32 (the reference's own log_softmax runs in bf16, quirk Q4);
 * entropy[r] = -sum_v p_v log p_v over the same distribution.  Either output may be NULL.  V % 256 == 0, K % 64 == 0. */
typedef struct {
  const void* x; const void* W;
  const int64_t* targets;
  float* logprobs; float* entropy;
  int64_t M; int V; int64_t K;
  void* workspace; size_t workspace_bytes;     /* evo_unembed_score_workspace(M, V) bytes */
} evo_score_params;
size_t evo_unembed_score_workspace(int64_t M, int V);
int evo_unembed_score(const evo_score_params* p, void* stream);

/* ==== models with an fp32 residual stream (Zaverax): row kernels, gated linear recurrence, windowed multi-map attention,
 * and an all-fp32 linear layer.  `dtype` arguments: 0 = bf16 activations, 1 = fp32 activations (the all-fp32 mode).
 * Weights and small parameter vectors are always bf16 as stored in the checkpoint. ==== */

/* table (vocab, D) bf16 -> out (n, D) fp32 */
int evo_embed_f32(const void* ids, int ids_are_i64, const void* table, float* out, int64_t n_tokens, int D, int vocab, void* stream);

/* Residual update + RMS norm in one pass over a row:
 *   x_row <- x_row + y_scale * y_row + add_row   (fp32, written back when y or x_add is given and gather is NULL)
 *   out_row = x_row / sqrt(mean(x_row^2) + eps) * (weight_offset + weight)        (weight NULL: no weight)
 * Output rows are laid out (B, halo + seq_len, ldo): the first `halo` rows of each sequence are copies of halo_src
 * (B, halo, D) fp32 (zeros when NULL) -- the carried inputs of a causal convolution that reads this output.
 * gather (B*seq_len) int64: read row gather[i] instead of row i (no write-back); used to norm only the rows whose logits are wanted.
 * Pad columns [D, ldo) of out are zero-filled. */
typedef struct {
  float* x;
  const void* y; int64_t ldy; int y_dtype; float y_scale;
  const float* x_add;
  const void* weight; float weight_offset; float eps;
  void* out; int64_t ldo; int out_dtype;
  int B; int64_t seq_len; int64_t halo; int D;
  const float* halo_src;
  const int64_t* gather;
} evo_resid_norm_params;
int evo_resid_norm(const evo_resid_norm_params* p, void* stream);

/* Per-channel causal convolution over time with a skip path: in (B, taps-1 + seq_len, D) fp32 whose first taps-1 rows are the
 * carried inputs; out[b,t,:] = in[b,taps-1+t,:] + sum_j weight[:,j] * in[b,t+j,:]; weight (D, taps) bf16.
 * carry_out (B, taps-1, D) fp32 (optional) receives the last taps-1 input rows. */
typedef struct {
  const float* in; const void* weight;
  void* out; int64_t ldo; int out_dtype;
  float* carry_out;
  int B; int64_t seq_len; int D; int taps;
} evo_causal_conv_params;
int evo_causal_conv(const evo_causal_conv_params* p, void* stream);

/* PolyNorm: out = a N(z) + b N(z^2) + c N(z^3) + e, N(u) = u / sqrt(mean(u^2) + eps) per row; coef = (a, b, c, e) bf16. */
int evo_polynorm(const void* z, int64_t ldz, const void* coef, void* out, int64_t ldo, int64_t rows, int F, float eps, int dtype, void* stream);
/* out (rows, V) fp32 = cap * tanh(in / cap)  (cap <= 0: plain copy) */
int evo_softcap_logits(const void* in, int64_t ldi, float* out, int64_t rows, int V, float cap, int dtype, void* stream);
/* rows of `width` elements: src row b*L + t -> dst + b*dst_batch_stride + (pos + t)*ldd, pos = *pos_dev if given else pos0 */
int evo_copy_rows(const void* src, int64_t lds, void* dst, int64_t ldd, int64_t dst_batch_stride, int B, int64_t L, int width,
                  int64_t pos0, const int64_t* pos_dev, int dtype, void* stream);

/* Gated linear recurrence (HGRN2): per head, with the raw projections q, f, v of a row,
 *   qa = silu(q), g = lower + (1 - lower) * sigmoid(f + f_bias),  S <- diag(g) S + (1 - g) v^T,  o = S^T qa,
 *   out = o / sqrt(mean(o^2) + eps) * norm_w   over the head's dv values.
 * S (B, H, dk, dv) fp32 is read (unless zero_start) and written back (unless NULL).  q/f/v may point into one fused buffer (row stride ld). */
typedef struct {
  const void* q; const void* f; const void* v; int64_t ld;
  const void* f_bias; const void* lower; const void* norm_w;
  float eps;
  float* state; int zero_start;
  void* out; int64_t ldo; int dtype;
  int B; int64_t L; int H, dk, dv;
} evo_hgrn2_params;
/* workspace: evo_hgrn2_workspace() bytes (0 unless a head's state is too large for one CTA and is split by value channel) */
size_t evo_hgrn2_workspace(const evo_hgrn2_params* p);
int evo_hgrn2_fwd(const evo_hgrn2_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Softmax attention over a linear key/value cache with a sliding window that keeps the first tokens, n_maps (1 or 2) score
 * maps per head over the same values (differential attention: o = a1 - lambda * a2), an optional per-head RMS norm without
 * weight times out_scale, and an optional sigmoid gate on the output.
 *   query row i of a sequence sits at position pos + i (pos = *pos_dev if given, else q_pos0) and sees key j iff
 *   j <= pos + i and (pos + i - j < window or j < keep_first); window <= 0 means plain causal.
 *   q: head h, map m at columns (h*n_maps + m)*dk; k: kv head g, map m at (g*n_maps + m)*dk; v: kv head g at g*dv;
 *   query head h reads kv head h / (H/G).  Scores, softmax weights and the combination are fp32. */
typedef struct {
  const void* q; int64_t q_tok_stride;
  const void* k; const void* v; int64_t k_tok_stride, v_tok_stride, k_batch_stride, v_batch_stride;
  const void* gate; int64_t gate_tok_stride;
  void* out; int64_t ldo; int dtype;
  int B; int64_t Lq; int H, G, dk, dv, n_maps;
  int64_t q_pos0; const int64_t* pos_dev;
  int64_t window, keep_first;
  float scale, lambda;
  int head_norm; float norm_eps, out_scale;
  int gate_per_head;      /* 1: gate holds one number per head (column h), else one per output channel (column h*dv + c) */
  /* optional extensions (all off when zero / NULL):
   *   softcap > 0: score <- softcap * tanh(score * scale / softcap);
   *   sink (H, bf16): exp(sink_h) joins every softmax denominator of head h (no key, no value, neither scaled nor capped);
   *   pool > 0: besides its window, query i sees one pooled key/value per block of `pool` tokens that lies wholly before the
   *   window, i.e. blocks b < (i - window + 1) / pool; pooled row b of a sequence is at pool_k/pool_v + batch * pool_batch_stride
   *   + b * pool_tok_stride with the column layout of k / v (the caller keeps them: evo_pool_rows).  Tokens and blocks share one softmax. */
  float softcap;
  const void* sink;
  int64_t pool;
  const void* pool_k; const void* pool_v; int64_t pool_tok_stride, pool_batch_stride;
  /*   dist_r1, dist_r2 (H, bf16; both or neither): a bias that grows with the distance is taken off the scaled (and capped) score of
   *   key j for query i: score <- score - r1_h * ln(1 + r2_h * (i - j)). */
  const void* dist_r1; const void* dist_r2;
} evo_window_attn_params;
int evo_window_attn_fwd(const evo_window_attn_params* p, void* stream);

/* C (M, N) = A (M, K) . W (N, K)^T with fp32 multiply-add on the CUDA cores (no tensor-core rounding): the linear layer of the
 * all-fp32 mode, and a shape-agnostic comparator for the bf16 one.  A and C have `dtype`; W is bf16. */
int evo_gemm_simt(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, int dtype, void* stream);

/* ==== designs whose branches are gated and normed on both sides, with latent attention, a minimal gated recurrence and
 * expert mixtures (Movalorn).  Same conventions: `dtype` 0 = bf16 activations, 1 = fp32; weights and parameter vectors bf16. ==== */

/* out (B*L, D) fp32 = table[id] * scale + pair[(prev * mul_prev + id * mul_cur) mod buckets]; a sequence without a previous token
 * uses pair row `buckets`.  prev_state (B) int64 (optional): the token before this call's first one (-1: none); the call leaves the
 * sequence's last token there. */
int evo_embed_pair_f32(const void* ids, int ids_are_i64, const void* table, const void* pair, float* out, int64_t* prev_state,
                       int B, int64_t L, int D, int vocab, float scale, int64_t buckets, int64_t mul_prev, int64_t mul_cur, void* stream);

/* Closes one branch and opens the next, one pass per row of the fp32 stream x (rows, D):
 *   u = y * sigmoid(gate + gate_bias)          (gate NULL: u = y)
 *   u = u / sqrt(mean(u^2) + eps) * post_gain   (post_norm)
 *   x <- x + u + row_add                        (replace: x <- u + row_add; y NULL: x unchanged)
 *   out = x / sqrt(mean(x^2) + eps) * gain      (concat: out = [x | cat] cast, no norm; out NULL: nothing)
 * gather (rows) int64: row i of out comes from stream row gather[i] and x is not written back.  Pad columns of out are zero. */
typedef struct {
  float* x;
  const void* y; int64_t ldy;
  const void* gate; int64_t ldg; const void* gate_bias;
  int post_norm; float post_gain;
  int replace; const void* row_add;
  float gain, eps;
  void* out; int64_t ldo;
  int concat; const float* cat;
  int dtype;
  int64_t rows; int D;
  const int64_t* gather;
} evo_branch_norm_params;
int evo_branch_norm(const evo_branch_norm_params* p, void* stream);

/* out[r, c] = act(gate[r, c]) * up[r, c] * w,  act 0 = tanh-form gelu, 1 = silu, 2 = erf-form gelu;  up NULL: no second factor;
 * w = group_w[r * ldw + c / group] for c < n_groups * group (fp32; NULL: 1) -- the weights of an expert mixture computed densely --
 * and for the columns after the groups w = group_w[r * ldw + n_groups] if tail_w is set, else 1; columns [F, ldo) are zero. */
int evo_glu_act(const void* gate, const void* up, int64_t ld, void* out, int64_t ldo, int64_t rows, int F, int act,
                const float* group_w, int64_t ldw, int group, int n_groups, int tail_w, int dtype, void* stream);
/* out (rows, V) fp32 = in * mul */
int evo_scale_logits(const void* in, int64_t ldi, float* out, int64_t rows, int V, float mul, int dtype, void* stream);

/* minGRU: per channel, with the raw projections z, u, g of a row (one fused buffer, row stride ld),
 *   a = sigmoid(z + z_bias), c = u + u_bias, cand = c + 1/2 (c >= 0) | sigmoid(c) (c < 0),  S <- (1 - a) S + a cand,  out = S * silu(g).
 * S (B, W) fp32 is read (unless zero_start) and written back (unless NULL); gates, candidate and state are fp32.
 * Long sequences are scanned in chunks (chunk products first, then each chunk from its carried-in state):
 * workspace evo_mingru_workspace() bytes. */
typedef struct {
  const void* z; const void* u; const void* g; int64_t ld;
  const void* z_bias; const void* u_bias;
  float* state; int zero_start;
  void* out; int64_t ldo; int dtype;
  int B; int64_t L; int W;
} evo_mingru_params;
size_t evo_mingru_workspace(const evo_mingru_params* p);
int evo_mingru_fwd(const evo_mingru_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Latent attention, preparation of a row of projections: the rotated part of every query head is turned in place, the first
 * `rank` entries of the down projection are RMS-normed (weight `norm_w`) into the latent, its last `rot` entries are turned, and
 * [latent | zeros up to rank_pad | rotated key part] is written to the cache row of the token's position
 * (pos = *pos_dev if given else pos0, plus the token's index).  Pairs (2i, 2i+1), 2i < rot_dims, turn by pos * freq[i] (freq fp32, rot_dims/2 entries). */
typedef struct {
  void* q; int64_t ldq;                       /* (B*L, H*(dim+rot)) in place */
  const void* dkv; int64_t ld_dkv;            /* (B*L, rank+rot) */
  const void* norm_w; float eps;
  const float* freq;
  void* cache; int64_t cache_row, cache_batch_stride; int rank_pad;
  int B; int64_t L; int H, dim, rot, rank;
  int64_t pos0; const int64_t* pos_dev; int dtype;
  int rot_dims;                               /* leading entries of a rotated part that are turned (even, <= rot) */
} evo_latent_prep_params;
int evo_latent_prep(const evo_latent_prep_params* p, void* stream);

/* Latent attention for few query rows (the decoding step) straight from the latent cache, in the absorbed form:
 *   ql = Uk_h^T q_a (rank),  s_j = (ql . c_j + q_b . kr_j) * scale over the visible j,  w = softmax(s),
 *   o = Uv_h (sum_j w_j c_j),  out_h = o * sigmoid(gate_h);   key j is visible from i iff 0 <= i - j < window (window <= 0: j <= i).
 * Everything between the bf16 (or fp32) inputs and the output is fp32. */
typedef struct {
  const void* q; int64_t ldq;                 /* prepared queries (B*Lq, H*(dim+rot)) */
  const void* cache; int64_t cache_row, cache_batch_stride; int rank_pad;
  const void* uk; const void* uv;             /* (H*dim, rank), (H*vdim, rank) bf16 */
  const void* gate; int64_t ld_gate;          /* (B*Lq, H) raw, optional */
  void* out; int64_t ldo;
  int B; int64_t Lq; int H, dim, rot, rank, vdim;
  int64_t pos0; const int64_t* pos_dev; int64_t window; float scale; int dtype;
  int64_t max_keys;                           /* host bound on the keys a query can see (sizes the key splits); 0: unknown */
} evo_latent_decode_params;
/* workspace: evo_latent_attn_decode_workspace() bytes (absorbed queries and per-split partial sums); with less, the per-head kernel runs */
size_t evo_latent_attn_decode_workspace(const evo_latent_decode_params* p);
int evo_latent_attn_decode(const evo_latent_decode_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Expert router: logits = W (E, D) . h in fp32, s = softmax(logits), the `top` experts with the largest s + correction are chosen;
 * weights (rows, E) fp32 = s * scale for the chosen experts, 0 for the others; chosen (rows, top) int32 (optional). */
int evo_moe_route(const void* h, int64_t ldh, const void* router_w, const void* correction, float* weights, int32_t* chosen,
                  int64_t rows, int D, int E, int top, float scale, int dtype, void* stream);
/* The router in general form.  logits = W . h in fp32 over E + n_extra rows of router_w (E experts, then n_extra further rows);
 *   score_fn 0: s = softmax over the experts, 1: s = sigmoid per expert;   choice score c = s + correction;
 *   groups > 1: the experts form `groups` equal runs of neighbours, a run's rank is the sum of its two largest c (of its one, when a run
 *   has one expert), and only experts of the `keep` best runs can be chosen;   the `top` largest c are chosen (ties: lower index);
 *   weights[r * ldw + e] = s_e * scale, or with normalize s_e / (sum of the chosen s + norm_eps) * scale; 0 for experts not chosen;
 *   weights[r * ldw + E + x] = sigmoid(logit of extra row x)   (gates that ride along, e.g. of an always-on expert). */
typedef struct {
  const void* h; int64_t ldh; const void* router_w; const void* correction;
  float* weights; int64_t ldw; int32_t* chosen;
  int64_t rows; int D, E, top, n_extra;
  int score_fn, groups, keep, normalize; float norm_eps, scale; int dtype;
} evo_moe_route_params;
int evo_moe_route_ex(const evo_moe_route_params* p, void* stream);
/* Sparse execution of the chosen experts.  chosen (n = rows * top) int32:
 *   evo_moe_count    counts[e] += 1 per entry (counts zeroed by the caller);
 *   evo_moe_scatter  slot_of[i] = offsets[chosen[i]] + running cursor (cursor zeroed by the caller), perm[slot] = i / top;
 *   evo_gather_rows  dst row r = src row perm[r] (rows of width_bytes, all strides and bases multiples of 16 bytes);
 *   evo_moe_combine  out[t] = g base[t] + sum_k weights[t*ldw + chosen[t,k]] * ys[slot_of[t,k]]  (fp32 sums, base optional, pad columns zero;
 *                    g = weights[t*ldw + E] if base_w is set, else 1). */
int evo_moe_count(const int32_t* chosen, int64_t n, int E, int32_t* counts, void* stream);
int evo_moe_scatter(const int32_t* chosen, int64_t n, int top, int E, const int32_t* offsets, int32_t* cursor, int32_t* perm, int32_t* slot_of, void* stream);
int evo_gather_rows(const void* src, int64_t ld_src_bytes, void* dst, int64_t ld_dst_bytes, const int32_t* perm, int64_t rows, int64_t width_bytes, void* stream);
int evo_moe_combine(const void* ys, int64_t ldy, const void* base, int64_t ldb, const float* weights, int64_t ldw, int base_w, const int32_t* chosen, const int32_t* slot_of,
                    void* out, int64_t ldo, int64_t rows, int D, int E, int top, int dtype, void* stream);

/* ==== designs whose layers run the mixer and the feed-forward side by side on two norms of the same stream, with matrix-state
 * recurrences (gated delta rule, state-space duality) and a windowed attention over tokens and pooled blocks (Nelovik).
 * Same conventions: `dtype` 0 = bf16 activations, 1 = fp32; weights and parameter vectors bf16. ==== */

/* Closes a layer of up to EVO_SUM_NORM_BRANCHES parallel branches and opens the next one, one pass per row of the fp32 stream x (rows, D):
 *   x <- x + sum_b scale[b] * (norm_w[b] ? y[b] / sqrt(mean(y[b]^2) + eps) * norm_w[b] : y[b])
 *   out[n] = x / sqrt(mean(x^2) + eps) * w[n]      for the outputs that are given (n < 2), pad columns [D, ldo) zero.
 * gather (rows) int64: row i reads stream row gather[i] (the branches are then added for the outputs only; x is not written back). */
#define EVO_SUM_NORM_BRANCHES 3
typedef struct {
  float* x;
  const void* y[EVO_SUM_NORM_BRANCHES]; int64_t ldy[EVO_SUM_NORM_BRANCHES];
  const void* norm_w[EVO_SUM_NORM_BRANCHES]; float scale[EVO_SUM_NORM_BRANCHES];
  int n_branches;
  float eps;
  void* out[2]; const void* w[2]; int64_t ldo;
  int dtype;
  int64_t rows; int D;
  const int64_t* gather;
} evo_sum_norm_params;
int evo_sum_norm(const evo_sum_norm_params* p, void* stream);

/* Short causal convolution over time per channel on columns of a projection, then an activation:
 *   out[b,t,c] = act(bias[c] + sum_j weight[c,j] * in[b, t - (taps-1) + j, c]),  act 0 = none, 1 = silu;
 * in (B*L, ld) rows, channel c at column c; weight (C, taps) bf16, the last column multiplies the current token; bias (C) bf16 optional.
 * carry (B, taps-1, C) fp32 (optional) holds the inputs before this call's first token (zero_start: zeros) and receives the last taps-1 inputs. */
typedef struct {
  const void* in; int64_t ld;
  const void* weight; const void* bias;
  float* carry; int zero_start;
  void* out; int64_t ldo;
  int B; int64_t L; int C, taps, act, dtype;
} evo_conv_act_params;
int evo_conv_act(const evo_conv_act_params* p, void* stream);

/* xIELU: out = softplus(p) z^2 + z/2 (z > 0), (1/2 + softplus(q)) (e^z - 1 - z) + z/2 (z <= 0); coef = (p, q) bf16; columns [F, ldo) zero. */
int evo_xielu(const void* z, int64_t ldz, const void* coef, void* out, int64_t ldo, int64_t rows, int F, int dtype, void* stream);

/* out = group_rms(y * silu(gate)) * norm_w: the row's `width` values are normed in `groups` equal parts, each by its own root mean
 * square; y (rows, width) fp32, gate (rows, ldg) and out (rows, ldo) activations, columns [width, ldo) zero. */
int evo_gated_group_norm(const float* y, const void* gate, int64_t ldg, const void* norm_w, void* out, int64_t ldo,
                         int64_t rows, int width, int groups, float eps, int dtype, void* stream);

/* Gated delta rule, per head h (key head h / (H/G)), over the activated projections q, k (G*dk), v (H*dv) of a row:
 *   qn = q / sqrt(sum(q^2) + unit_eps) * q_scale,  kn = k / sqrt(sum(k^2) + unit_eps),
 *   beta = sigmoid(b_h),  g = exp(-exp(A_log_h) * softplus(a_h + dt_bias_h)),
 *   S <- g S;  u = beta (v - S^T kn);  S <- S + kn u^T;  o = S^T qn,
 *   out = o / sqrt(mean(o^2) + eps) * norm_w * silu(gate)     over the head's dv values.
 * S (B, H, dk, dv) fp32 is read (unless zero_start) and written back (unless NULL); everything after the inputs is fp32. */
typedef struct {
  const void* q; const void* k; const void* v; int64_t ld;         /* one buffer of activated projections, row stride ld */
  const void* b; const void* a; const void* gate; int64_t ldz;    /* raw projections: (rows, H), (rows, H), (rows, H*dv), row stride ldz */
  const void* A_log; const void* dt_bias; const void* norm_w;
  float eps, unit_eps, q_scale;
  float* state; int zero_start;
  void* out; int64_t ldo; int dtype;
  int B; int64_t L; int H, G, dk, dv;
} evo_gated_delta_params;
/* workspace: evo_gated_delta_workspace() bytes (0 unless a head's value channels are spread over several CTAs; the head norm then runs in a second kernel) */
size_t evo_gated_delta_workspace(const evo_gated_delta_params* p);
int evo_gated_delta_fwd(const evo_gated_delta_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* State-space duality recurrence, per head h (group h / (H/G)), over the activated x (H*dv), Bm, Cm (G*N) of a row and the raw step dt (H):
 *   d = softplus(dt_h + dt_bias_h),  S <- exp(-exp(A_log_h) d) S + d Bm x^T,  y = S^T Cm + D_h x     (S is N x dv, fp32).
 * y (rows, H*dv) fp32.  S (B, H, N, dv) fp32 is read (unless zero_start) and written back (unless NULL). */
typedef struct {
  const void* x; const void* Bm; const void* Cm; int64_t ld;
  const void* dt; int64_t ld_dt;
  const void* A_log; const void* dt_bias; const void* D;
  float* state; int zero_start;
  float* y;
  int dtype;
  int B; int64_t L; int H, G, N, dv;
} evo_ssd_params;
int evo_ssd_fwd(const evo_ssd_params* p, void* stream);

/* Preparation of attention projections whose query and key are normed (over the WHOLE projection unless norm_per_head) and partly rotated, one row at a time:
 *   q <- rms(q + q_bias) * q_norm_w (over all H*dk entries), k likewise over G*dk, v <- v + v_bias;
 *   in every head the first rot_dims entries turn by pos * freq[i], entry i paired with entry i + rot_dims/2 (i < rot_dims/2; freq fp32);
 *   q is written back in place, [k | v] goes to the cache row of the token's position (pos = *pos_dev if given else pos0, plus its index). */
typedef struct {
  void* q; const void* k; const void* v; int64_t ld;                /* one projection buffer (rows, ld) */
  const void* q_bias; const void* k_bias; const void* v_bias;     /* optional */
  const void* q_norm_w; const void* k_norm_w; float eps;
  const float* freq; int rot_dims;
  void* cache; int64_t cache_row, cache_batch_stride;
  int B; int64_t L; int H, G, dk, dv;
  int64_t pos0; const int64_t* pos_dev; int dtype;
  /* optional extensions (off when zero):
   *   norm_per_head: the norms run over each head's dk entries and q_norm_w / k_norm_w hold dk entries shared by all heads;
   *   q_temp_every > 0: after norm and rotation the query is multiplied by 1 + q_temp_coef * ln(pos / q_temp_every + 1), with the
   *   integer quotient of (pos + 1) -- a query temperature that grows with the position in steps of q_temp_every tokens. */
  int norm_per_head;
  float q_temp_coef; int64_t q_temp_every;
} evo_qk_prep_params;
int evo_qk_prep(const evo_qk_prep_params* p, void* stream);

/* Pooled cache rows: for every block b of `pool` consecutive cache rows that this call completed (its last row bP + P - 1 lies in
 * [pos, pos + L)), pooled row b = mean of the block's rows as the cache holds them (fp32 sum), `width` entries per row. */
int evo_pool_rows(const void* cache, int64_t cache_row, int64_t cache_batch_stride, void* pooled, int64_t pooled_row, int64_t pooled_batch_stride,
                  int B, int64_t L, int width, int64_t pool, int64_t pos0, const int64_t* pos_dev, int dtype, void* stream);

/* ==== designs that norm the OUTPUT of every sublayer (layer norm with weight and bias) before it joins the fp32 stream, whose sublayers
 * read the stream itself, and that hand on a learned mix of all earlier layers' results (Gakupel). ==== */

/* One row kernel between two sublayers:
 *   t = sum_b scale[b] * y[b]                      (n_in <= 2 sublayer outputs of the activation type, fp32 sum)
 *   x <- x + ln(t; norm_w, norm_b)                 (skipped when n_in == 0;  ln(u) = (u - mean) / sqrt(var + eps) * w + b, biased variance)
 *   mix_n > 0:  stack[mix_n - 1] <- x;  x <- sum_{j < mix_n} mix_w[j] * stack[j]      (stack (slots, rows, D) fp32, slot stride stack_stride)
 *   out <- x, or ln(x; out_norm_w, out_norm_b) when out_norm_w is given, in the activation type, columns [D, ldo) zero
 * x is read from x_in (default: x) and written to x; with `gather` (row indices) only those rows are read and nothing but `out` is written. */
typedef struct {
  float* x; const float* x_in;
  const void* y[2]; int64_t ldy[2]; float scale[2]; int n_in;
  const void* norm_w; const void* norm_b; float eps;
  float* stack; int64_t stack_stride; int mix_n; const void* mix_w;
  void* out; int64_t ldo; const void* out_norm_w; const void* out_norm_b;
  int dtype; int64_t rows; int D; const int64_t* gather;
} evo_post_norm_params;
int evo_post_norm(const evo_post_norm_params* p, void* stream);

/* Matrix memory with exponential gates kept stable by a running maximum (mLSTM), per head h over q, k (H*dk) and v (H*dv) of a row and
 * the raw gate projections gi, gf (H):   i = cap tanh((gi + i_bias) / cap),  f = logsigmoid(cap tanh((gf + f_bias) / cap))   (cap <= 0: no cap)
 *   m' = max(f + m, i);  S <- e^{f + m - m'} S + e^{i - m'} k v^T;  n likewise with k;  o = S^T (q q_scale) / (max(|n . q q_scale|, e^{-m'}) + den_eps)
 *   out = o / sqrt(mean_c o^2 + eps) * norm_w[h*dv + c] * sigmoid(gate[h*dv + c])
 * state (B, H, dk * dv + dk) fp32: S (dk x dv), then n; mstate (B, H) fp32: m (zero_start: all start at 0).
 * workspace: evo_mlstm_workspace() bytes (0 unless a head's value channels are spread over several CTAs). */
typedef struct {
  const void* q; const void* k; const void* v; int64_t ld;
  const void* gi; const void* gf; int64_t ldg;
  const void* i_bias; const void* f_bias; float cap, q_scale, den_eps;
  const void* gate; int64_t ld_gate; const void* norm_w; float eps;
  float* state; float* mstate; int zero_start;
  void* out; int64_t ldo; int dtype;
  int B; int64_t L; int H, dk, dv;
} evo_mlstm_params;
size_t evo_mlstm_workspace(const evo_mlstm_params* p);
int evo_mlstm_fwd(const evo_mlstm_params* p, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif
