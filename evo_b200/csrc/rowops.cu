// Row-wise kernels for models that keep the residual stream in fp32: embedding gather into fp32, residual update +
// RMS norm in one pass (with an optional halo of carried rows for a short causal convolution that follows), the
// per-channel causal convolution itself, the PolyNorm activation, the tanh soft cap of the logits and a strided row copy
// (cache append).  Activations that feed a GEMM are written in the GEMM's input type (bf16, or fp32 for the all-fp32
// mode) with the pad columns [D, ld) zero-filled, so that K can be padded to the tensor-core tile without a second pass.
// All statistics (mean squares, reciprocal roots, polynomial terms, tanh) are fp32.
#include "common.cuh"
#include "../../include/evo_b200.h"

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// 4 consecutive elements as floats (16-byte / 8-byte accesses; the callers check alignment and divisibility)
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf_lo(u.x), bf_hi(u.x), bf_lo(u.y), bf_hi(u.y));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) { *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w)); }
inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
inline bool aligned_to(const void* p, int n) { return ((uintptr_t)p & (uintptr_t)(n - 1)) == 0; }

// sum over the block (blockDim.x <= 1024, a multiple of 32); every thread gets the total
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();                      // red may still be read from a previous call
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// ------------------------------------------------------------------ embedding gather into the fp32 stream
template <typename IdT>
__global__ void embed_f32_kernel(const IdT* __restrict__ ids, const bf16* __restrict__ table, float* __restrict__ out,
                                 int64_t n_tokens, int D, int vocab) {
  const int64_t row = blockIdx.x;
  long long id = (long long)ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const bf16* src = table + (int64_t)id * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) out[row * D + c] = __bfloat162float(src[c]);
}

// ------------------------------------------------------------------ residual update + RMS norm
// One CTA per output row.  Output rows are laid out (B, halo + L, .): rows t < halo of a sequence are copies of carried
// rows (or zeros); the others are norm(x_row) with x_row <- x_row + y_scale * y_row + add_row written back first.
template <typename TY, typename TO, bool VEC>
__global__ void __launch_bounds__(256) resid_norm_kernel(evo_resid_norm_params p) {
  __shared__ float red[32];
  const int64_t per = p.halo + p.seq_len;
  const int64_t r = blockIdx.x;
  const int64_t b = r / per, t = r % per - p.halo;
  TO* orow = (TO*)p.out + r * p.ldo;
  const int D = p.D;
  if (t < 0) {
    const float* src = p.halo_src ? p.halo_src + (b * p.halo + (t + p.halo)) * (int64_t)D : nullptr;
    for (int c = threadIdx.x; c < p.ldo; c += blockDim.x) stf(orow + c, (src && c < D) ? src[c] : 0.f);
    return;
  }
  const int64_t srow = p.gather ? p.gather[b * p.seq_len + t] : b * p.seq_len + t;
  float* xr = p.x + srow * D;
  const TY* yr = p.y ? (const TY*)p.y + srow * p.ldy : nullptr;
  const float* ar = p.x_add ? p.x_add + srow * D : nullptr;
  const bool update = (yr != nullptr || ar != nullptr) && p.gather == nullptr;
  float ss = 0.f;
  if (VEC) {                              // D, ldy, ldo multiples of 4 and 16-byte aligned rows: 4 channels per access
    for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
      float4 v = ld4(xr + c);
      if (yr) { const float4 y4 = ld4(yr + c); v.x = fmaf(p.y_scale, y4.x, v.x); v.y = fmaf(p.y_scale, y4.y, v.y); v.z = fmaf(p.y_scale, y4.z, v.z); v.w = fmaf(p.y_scale, y4.w, v.w); }
      if (ar) { const float4 a4 = ld4(ar + c); v.x += a4.x; v.y += a4.y; v.z += a4.z; v.w += a4.w; }
      if (update) st4(xr + c, v);
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)D + p.eps);
    const bf16* w = (const bf16*)p.weight;
    for (int c = threadIdx.x * 4; c < p.ldo; c += blockDim.x * 4) {
      float4 h = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < D) {
        float4 v = ld4(xr + c);
        if (!update) {
          if (yr) { const float4 y4 = ld4(yr + c); v.x = fmaf(p.y_scale, y4.x, v.x); v.y = fmaf(p.y_scale, y4.y, v.y); v.z = fmaf(p.y_scale, y4.z, v.z); v.w = fmaf(p.y_scale, y4.w, v.w); }
          if (ar) { const float4 a4 = ld4(ar + c); v.x += a4.x; v.y += a4.y; v.z += a4.z; v.w += a4.w; }
        }
        h = make_float4(v.x * rstd, v.y * rstd, v.z * rstd, v.w * rstd);
        if (w) { const float4 w4 = ld4(w + c); h.x *= p.weight_offset + w4.x; h.y *= p.weight_offset + w4.y; h.z *= p.weight_offset + w4.z; h.w *= p.weight_offset + w4.w; }
      }
      st4(orow + c, h);
    }
    return;
  }
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float v = xr[c];
    if (yr) v = fmaf(p.y_scale, ldf(yr + c), v);
    if (ar) v += ar[c];
    if (update) xr[c] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(ss / (float)D + p.eps);
  const bf16* w = (const bf16*)p.weight;
  for (int c = threadIdx.x; c < p.ldo; c += blockDim.x) {
    float h = 0.f;
    if (c < D) {
      float v = xr[c];
      if (!update) {                      // nothing was written back: rebuild the value
        if (yr) v = fmaf(p.y_scale, ldf(yr + c), v);
        if (ar) v += ar[c];
      }
      h = v * rstd;
      if (w) h *= p.weight_offset + __bfloat162float(w[c]);
    }
    stf(orow + c, h);
  }
}

// ------------------------------------------------------------------ per-channel causal convolution with a skip path
// in (B, taps-1 + L, D) fp32: the first taps-1 rows of a sequence are the carried inputs.  out[b,t,c] = in[b,taps-1+t,c] +
// sum_j w[c,j] * in[b,t+j,c]; the last taps-1 input rows become the next carried rows.
template <typename TO, bool VEC>
__global__ void __launch_bounds__(256) causal_conv_kernel(evo_causal_conv_params p) {
  const int halo = p.taps - 1;
  const int64_t per = p.seq_len + halo;
  const int64_t r = blockIdx.x;
  const int64_t b = r / per, t = r % per;
  const float* in = p.in + b * per * (int64_t)p.D;
  const bf16* w = (const bf16*)p.weight;
  if (t >= p.seq_len) {                   // carried rows for the next call
    if (!p.carry_out) return;
    const int64_t k = t - p.seq_len;
    for (int c = threadIdx.x; c < p.D; c += blockDim.x) p.carry_out[(b * halo + k) * (int64_t)p.D + c] = in[(p.seq_len + k) * (int64_t)p.D + c];
    return;
  }
  TO* orow = (TO*)p.out + (b * p.seq_len + t) * p.ldo;
  if (VEC) {                              // D and ldo multiples of 4, 16-byte aligned rows: 4 channels per access
    for (int c = threadIdx.x * 4; c < p.ldo; c += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < p.D) {
        acc = ld4(in + (t + halo) * (int64_t)p.D + c);
        for (int j = 0; j < p.taps; ++j) {
          const float4 v = ld4(in + (t + j) * (int64_t)p.D + c);
          const bf16* wc = w + (int64_t)c * p.taps + j;
          acc.x = fmaf(__bfloat162float(wc[0]), v.x, acc.x);
          acc.y = fmaf(__bfloat162float(wc[p.taps]), v.y, acc.y);
          acc.z = fmaf(__bfloat162float(wc[2 * p.taps]), v.z, acc.z);
          acc.w = fmaf(__bfloat162float(wc[3 * p.taps]), v.w, acc.w);
        }
      }
      st4(orow + c, acc);
    }
    return;
  }
  for (int c = threadIdx.x; c < p.ldo; c += blockDim.x) {
    float acc = 0.f;
    if (c < p.D) {
      acc = in[(t + halo) * (int64_t)p.D + c];
      for (int j = 0; j < p.taps; ++j) acc = fmaf(__bfloat162float(w[(int64_t)c * p.taps + j]), in[(t + j) * (int64_t)p.D + c], acc);
    }
    stf(orow + c, acc);
  }
}

// ------------------------------------------------------------------ PolyNorm: a N(z) + b N(z^2) + c N(z^3) + e
// N divides a row by its root mean square; one CTA per row, two passes over the row (the second one hits L1/L2).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) polynorm_kernel(const T* __restrict__ z, int64_t ldz, const bf16* __restrict__ coef, T* __restrict__ out,
                                                       int64_t ldo, int F, float eps) {
  __shared__ float red[32];
  const T* zr = z + (int64_t)blockIdx.x * ldz;
  T* orow = out + (int64_t)blockIdx.x * ldo;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < F; c += blockDim.x * 4) {
      const float4 q = ld4(zr + c);
      const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float v = e[i], v2 = v * v, v3 = v2 * v; s1 = fmaf(v, v, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3); }
    }
  } else {
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
      const float v = ldf(zr + c), v2 = v * v, v3 = v2 * v;
      s1 = fmaf(v, v, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
    }
  }
  s1 = block_sum(s1, red); s2 = block_sum(s2, red); s3 = block_sum(s3, red);
  const float a = __bfloat162float(coef[0]) / sqrtf(s1 / (float)F + eps);
  const float b = __bfloat162float(coef[1]) / sqrtf(s2 / (float)F + eps);
  const float c3 = __bfloat162float(coef[2]) / sqrtf(s3 / (float)F + eps);
  const float e = __bfloat162float(coef[3]);
  if (VEC) {
    for (int c = threadIdx.x * 4; c < ldo; c += blockDim.x * 4) {
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < F) {
        const float4 q = ld4(zr + c);
        o.x = fmaf(a, q.x, fmaf(b, q.x * q.x, fmaf(c3, q.x * q.x * q.x, e)));
        o.y = fmaf(a, q.y, fmaf(b, q.y * q.y, fmaf(c3, q.y * q.y * q.y, e)));
        o.z = fmaf(a, q.z, fmaf(b, q.z * q.z, fmaf(c3, q.z * q.z * q.z, e)));
        o.w = fmaf(a, q.w, fmaf(b, q.w * q.w, fmaf(c3, q.w * q.w * q.w, e)));
      }
      st4(orow + c, o);
    }
    return;
  }
  for (int c = threadIdx.x; c < ldo; c += blockDim.x) {
    float o = 0.f;
    if (c < F) {
      const float v = ldf(zr + c), v2 = v * v;
      o = fmaf(a, v, fmaf(b, v2, fmaf(c3, v2 * v, e)));
    }
    stf(orow + c, o);
  }
}

template <typename T>
__global__ void softcap_kernel(const T* __restrict__ in, int64_t ldi, float* __restrict__ out, int64_t rows, int V, float cap, float mul) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * V) return;
  const int64_t r = i / V; const int c = (int)(i % V);
  const float v = ldf(in + r * ldi + c);
  out[i] = mul * (cap > 0.f ? cap * tanhf(v / cap) : v);
}

// rows of `width` elements from src (row stride lds) to dst rows [pos, pos + L) of each sequence (row stride ldd, batch stride)
template <typename T>
__global__ void copy_rows_kernel(const T* __restrict__ src, int64_t lds, T* __restrict__ dst, int64_t ldd, int64_t dst_batch_stride,
                                 int B, int64_t L, int width, int64_t pos0, const long long* __restrict__ pos_dev) {
  const int64_t r = blockIdx.x;
  const int64_t b = r / L, t = r % L;
  const int64_t pos = (pos_dev ? (int64_t)*pos_dev : pos0) + t;
  const T* s = src + r * lds;
  T* d = dst + b * dst_batch_stride + pos * ldd;
  for (int c = threadIdx.x; c < width; c += blockDim.x) d[c] = s[c];
}

}  // namespace

extern "C" int evo_embed_f32(const void* ids, int ids_are_i64, const void* table, float* out, int64_t n_tokens, int D, int vocab, void* stream) {
  if (n_tokens == 0) return 0;
  dim3 grid((unsigned)n_tokens), block(128);
  if (ids_are_i64) embed_f32_kernel<long long><<<grid, block, 0, (cudaStream_t)stream>>>((const long long*)ids, (const bf16*)table, out, n_tokens, D, vocab);
  else embed_f32_kernel<int><<<grid, block, 0, (cudaStream_t)stream>>>((const int*)ids, (const bf16*)table, out, n_tokens, D, vocab);
  return check_launch("evo_embed_f32");
}

extern "C" int evo_resid_norm(const evo_resid_norm_params* p, void* stream) {
  EVO_REQUIRE(p->x && p->out && p->D > 0 && p->ldo >= p->D && p->B >= 0 && p->seq_len >= 0 && p->halo >= 0, "evo_resid_norm: bad arguments");
  EVO_REQUIRE(p->y == nullptr || p->ldy >= p->D, "evo_resid_norm: ldy < D");
  const int64_t rows = (int64_t)p->B * (p->halo + p->seq_len);
  if (rows == 0 || p->seq_len == 0) return 0;
  dim3 grid((unsigned)rows), block(p->D >= 1024 ? 256 : 128);
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = p->D % 4 == 0 && p->ldo % 4 == 0 && (p->y == nullptr || p->ldy % 4 == 0) && aligned16(p->x) && aligned16(p->out) && aligned16(p->y) &&
                   aligned16(p->x_add) && aligned16(p->weight) && aligned16(p->halo_src);
  const int key = (p->y_dtype ? 4 : 0) | (p->out_dtype ? 2 : 0) | (vec ? 1 : 0);
  switch (key) {
    case 0: resid_norm_kernel<bf16, bf16, false><<<grid, block, 0, st>>>(*p); break;
    case 1: resid_norm_kernel<bf16, bf16, true><<<grid, block, 0, st>>>(*p); break;
    case 2: resid_norm_kernel<bf16, float, false><<<grid, block, 0, st>>>(*p); break;
    case 3: resid_norm_kernel<bf16, float, true><<<grid, block, 0, st>>>(*p); break;
    case 4: resid_norm_kernel<float, bf16, false><<<grid, block, 0, st>>>(*p); break;
    case 5: resid_norm_kernel<float, bf16, true><<<grid, block, 0, st>>>(*p); break;
    case 6: resid_norm_kernel<float, float, false><<<grid, block, 0, st>>>(*p); break;
    default: resid_norm_kernel<float, float, true><<<grid, block, 0, st>>>(*p); break;
  }
  return check_launch("evo_resid_norm");
}

extern "C" int evo_causal_conv(const evo_causal_conv_params* p, void* stream) {
  EVO_REQUIRE(p->in && p->out && p->weight && p->D > 0 && p->taps >= 1 && p->ldo >= p->D && p->B >= 0 && p->seq_len >= 0, "evo_causal_conv: bad arguments");
  const int64_t rows = (int64_t)p->B * (p->seq_len + p->taps - 1);
  if (rows == 0) return 0;
  dim3 grid((unsigned)rows), block(p->D >= 1024 ? 256 : 128);
  const bool vec = p->D % 4 == 0 && p->ldo % 4 == 0 && aligned16(p->in) && aligned16(p->out);
  cudaStream_t st = (cudaStream_t)stream;
  if (p->out_dtype) { if (vec) causal_conv_kernel<float, true><<<grid, block, 0, st>>>(*p); else causal_conv_kernel<float, false><<<grid, block, 0, st>>>(*p); }
  else { if (vec) causal_conv_kernel<bf16, true><<<grid, block, 0, st>>>(*p); else causal_conv_kernel<bf16, false><<<grid, block, 0, st>>>(*p); }
  return check_launch("evo_causal_conv");
}

extern "C" int evo_polynorm(const void* z, int64_t ldz, const void* coef, void* out, int64_t ldo, int64_t rows, int F, float eps, int dtype, void* stream) {
  EVO_REQUIRE(z && out && coef && F > 0 && ldz >= F && ldo >= F, "evo_polynorm: bad arguments");
  if (rows == 0) return 0;
  dim3 grid((unsigned)rows), block(256);
  const bool vec = F % 4 == 0 && ldz % 4 == 0 && ldo % 4 == 0 && aligned16(z) && aligned16(out);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype) {
    if (vec) polynorm_kernel<float, true><<<grid, block, 0, st>>>((const float*)z, ldz, (const bf16*)coef, (float*)out, ldo, F, eps);
    else polynorm_kernel<float, false><<<grid, block, 0, st>>>((const float*)z, ldz, (const bf16*)coef, (float*)out, ldo, F, eps);
  } else {
    if (vec) polynorm_kernel<bf16, true><<<grid, block, 0, st>>>((const bf16*)z, ldz, (const bf16*)coef, (bf16*)out, ldo, F, eps);
    else polynorm_kernel<bf16, false><<<grid, block, 0, st>>>((const bf16*)z, ldz, (const bf16*)coef, (bf16*)out, ldo, F, eps);
  }
  return check_launch("evo_polynorm");
}

extern "C" int evo_softcap_logits(const void* in, int64_t ldi, float* out, int64_t rows, int V, float cap, int dtype, void* stream) {
  EVO_REQUIRE(in && out && V > 0 && ldi >= V, "evo_softcap_logits: bad arguments");
  if (rows == 0) return 0;
  const int64_t n = rows * V;
  dim3 grid((unsigned)((n + 255) / 256)), block(256);
  if (dtype) softcap_kernel<float><<<grid, block, 0, (cudaStream_t)stream>>>((const float*)in, ldi, out, rows, V, cap, 1.f);
  else softcap_kernel<bf16><<<grid, block, 0, (cudaStream_t)stream>>>((const bf16*)in, ldi, out, rows, V, cap, 1.f);
  return check_launch("evo_softcap_logits");
}

extern "C" int evo_copy_rows(const void* src, int64_t lds, void* dst, int64_t ldd, int64_t dst_batch_stride, int B, int64_t L, int width,
                             int64_t pos0, const int64_t* pos_dev, int dtype, void* stream) {
  EVO_REQUIRE(src && dst && width > 0 && lds >= width && ldd >= width, "evo_copy_rows: bad arguments");
  if ((int64_t)B * L == 0) return 0;
  dim3 grid((unsigned)((int64_t)B * L)), block(128);
  if (dtype) copy_rows_kernel<float><<<grid, block, 0, (cudaStream_t)stream>>>((const float*)src, lds, (float*)dst, ldd, dst_batch_stride, B, L, width, pos0, (const long long*)pos_dev);
  else copy_rows_kernel<bf16><<<grid, block, 0, (cudaStream_t)stream>>>((const bf16*)src, lds, (bf16*)dst, ldd, dst_batch_stride, B, L, width, pos0, (const long long*)pos_dev);
  return check_launch("evo_copy_rows");
}

// =====================================================================================================================
// Row kernels of the designs whose branches are normed on both sides and gated (Movalorn): token + hashed-pair embedding,
// the branch close / open kernel, the gated-linear-unit activation with an optional per-row weight per column group, and the
// final logit scaling.
namespace {

// out[row] = table[id] * scale + pair[(prev * mul_prev + id * mul_cur) mod buckets], pair row `buckets` when the sequence has no
// previous token (prev < 0).  prev of a sequence's first new token comes from prev_state[b]; the CTA of that token then stores the
// sequence's last new token there (it is the only CTA that touches prev_state[b]).
template <typename IdT>
__global__ void embed_pair_kernel(const IdT* __restrict__ ids, const bf16* __restrict__ table, const bf16* __restrict__ pair, float* __restrict__ out,
                                  long long* __restrict__ prev_state, int64_t L, int D, int vocab, float scale,
                                  long long buckets, long long mul_prev, long long mul_cur) {
  const int64_t row = blockIdx.x, b = row / L, t = row % L;
  auto clampid = [vocab](long long v) { return v < 0 ? 0LL : (v >= vocab ? (long long)vocab - 1 : v); };
  const long long id = clampid((long long)ids[row]);
  long long prev;
  if (t > 0) prev = clampid((long long)ids[row - 1]);
  else prev = prev_state ? prev_state[b] : -1;
  __syncthreads();
  if (t == 0 && prev_state && threadIdx.x == 0) prev_state[b] = clampid((long long)ids[b * L + L - 1]);
  const long long slot = prev < 0 ? buckets : (prev * mul_prev + id * mul_cur) % buckets;
  const bf16* src = table + (int64_t)id * D;
  const bf16* pr = pair + (int64_t)slot * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) out[row * D + c] = fmaf(__bfloat162float(src[c]), scale, __bfloat162float(pr[c]));
}

// sigmoid and the two gate activations: IEEE exp / tanh / division for fp32 activations (the all-fp32 mode), the hardware
// approximations (ex2, rcp: relative error ~1e-6) for bf16 activations, whose own rounding is 4e-3
template <typename T> __device__ __forceinline__ float sigm(float v);
template <> __device__ __forceinline__ float sigm<float>(float v) { return 1.f / (1.f + expf(-v)); }
template <> __device__ __forceinline__ float sigm<bf16>(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }

template <typename T>
__device__ __forceinline__ float gated_value(const T* yr, const T* gr, const bf16* gb, int c) {
  float u = ldf(yr + c);
  if (gr) u *= sigm<T>(ldf(gr + c) + (gb ? __bfloat162float(gb[c]) : 0.f));
  return u;
}

// One CTA per row:  u = y * sigmoid(gate + gate_bias);  u <- u / rms(u) * post_gain (post_norm);  x <- x + u  (or u + row_add when
// replace);  then out = x / rms(x) * gain, or (concat) out = [x | cat_row] cast without a norm.  All sums fp32.
// VEC: 4 channels per access (D and every row stride a multiple of 4 elements, 16-byte aligned bases).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) branch_norm_kernel(evo_branch_norm_params p) {
  __shared__ float red[32];
  const int64_t r = blockIdx.x;
  const int64_t srow = p.gather ? p.gather[r] : r;
  const int D = p.D;
  float* xr = p.x + srow * D;
  const T* yr = p.y ? (const T*)p.y + srow * p.ldy : nullptr;
  const T* gr = (p.y && p.gate) ? (const T*)p.gate + srow * p.ldg : nullptr;
  const bf16* gb = (const bf16*)p.gate_bias;
  const bf16* ra = (const bf16*)p.row_add;
  const bool write_back = p.gather == nullptr && (yr != nullptr || ra != nullptr);
  constexpr int VW = VEC ? 4 : 1;
  // u of channels [c, c + VW)
  auto gated = [&](int c, float* u) {
    if (VEC) {
      const float4 y4 = ld4(yr + c);
      u[0] = y4.x; u[1] = y4.y; u[2] = y4.z; u[3] = y4.w;
      if (gr) {
        const float4 g4 = ld4(gr + c);
        float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gb) b4 = ld4(gb + c);
        u[0] *= sigm<T>(g4.x + b4.x); u[1] *= sigm<T>(g4.y + b4.y); u[2] *= sigm<T>(g4.z + b4.z); u[3] *= sigm<T>(g4.w + b4.w);
      }
    } else {
      u[0] = gated_value(yr, gr, gb, c);
    }
  };
  float mul = 1.f;
  if (yr && p.post_norm) {
    float su = 0.f;
    for (int c = threadIdx.x * VW; c < D; c += blockDim.x * VW) {
      float u[VW];
      gated(c, u);
#pragma unroll
      for (int k = 0; k < VW; ++k) su = fmaf(u[k], u[k], su);
    }
    su = block_sum(su, red);
    mul = p.post_gain / sqrtf(su / (float)D + p.eps);
  }
  auto value = [&](int c, float* v) {
    if (p.replace) {
#pragma unroll
      for (int k = 0; k < VW; ++k) v[k] = 0.f;
    } else if (VEC) {
      const float4 x4 = ld4(xr + c);
      v[0] = x4.x; v[1] = x4.y; v[2] = x4.z; v[3] = x4.w;
    } else {
      v[0] = xr[c];
    }
    if (yr) {
      float u[VW];
      gated(c, u);
#pragma unroll
      for (int k = 0; k < VW; ++k) v[k] = fmaf(u[k], mul, v[k]);
    }
    if (ra) {
      if (VEC) { const float4 a4 = ld4(ra + c); v[0] += a4.x; v[1] += a4.y; v[2] += a4.z; v[3] += a4.w; }
      else v[0] += __bfloat162float(ra[c]);
    }
  };
  auto stream = [&](int c, float* v) {       // the row after the update: what this thread wrote back, else rebuilt
    if (!write_back) { value(c, v); return; }
    if (VEC) { const float4 x4 = ld4(xr + c); v[0] = x4.x; v[1] = x4.y; v[2] = x4.z; v[3] = x4.w; }
    else v[0] = xr[c];
  };
  float ss = 0.f;
  for (int c = threadIdx.x * VW; c < D; c += blockDim.x * VW) {
    float v[VW];
    value(c, v);
    if (write_back) {
      if (VEC) st4(xr + c, make_float4(v[0], v[1], v[2], v[3]));
      else xr[c] = v[0];
    }
#pragma unroll
    for (int k = 0; k < VW; ++k) ss = fmaf(v[k], v[k], ss);
  }
  if (!p.out) return;
  T* orow = (T*)p.out + r * p.ldo;
  float g = 1.f;
  const float* cr = p.concat ? p.cat + srow * D : nullptr;
  if (!p.concat) {
    ss = block_sum(ss, red);
    g = p.gain / sqrtf(ss / (float)D + p.eps);
  }
  for (int c = threadIdx.x * VW; c < p.ldo; c += blockDim.x * VW) {
    float v[VW];
#pragma unroll
    for (int k = 0; k < VW; ++k) v[k] = 0.f;
    if (c < D) {
      stream(c, v);
#pragma unroll
      for (int k = 0; k < VW; ++k) v[k] *= g;
    } else if (cr && c < 2 * D) {
      if (VEC) { const float4 c4 = ld4(cr + c - D); v[0] = c4.x; v[1] = c4.y; v[2] = c4.z; v[3] = c4.w; }
      else v[0] = cr[c - D];
    }
    if (VEC) st4(orow + c, make_float4(v[0], v[1], v[2], v[3]));
    else stf(orow + c, v[0]);
  }
}

// The same for rows of at most 16 x blockDim channels on the vector path: a thread keeps its (up to 16) channels in registers from the
// first read to the last store, so the branch, its gate and the stream are read once and every sigmoid is evaluated once.
template <typename T>
__global__ void __launch_bounds__(256) branch_norm_cached_kernel(evo_branch_norm_params p) {
  __shared__ float red[32];
  constexpr int NIT = 4;
  const int64_t r = blockIdx.x;
  const int64_t srow = p.gather ? p.gather[r] : r;
  const int D = p.D, step = blockDim.x * 4, c0 = threadIdx.x * 4;
  float* xr = p.x + srow * D;
  const T* yr = p.y ? (const T*)p.y + srow * p.ldy : nullptr;
  const T* gr = (p.y && p.gate) ? (const T*)p.gate + srow * p.ldg : nullptr;
  const bf16* gb = (const bf16*)p.gate_bias;
  const bf16* ra = (const bf16*)p.row_add;
  const bool write_back = p.gather == nullptr && (yr != nullptr || ra != nullptr);
  float c[NIT][4];
  float su = 0.f;
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    const int col = c0 + it * step;
    c[it][0] = c[it][1] = c[it][2] = c[it][3] = 0.f;
    if (yr && col < D) {
      const float4 y4 = ld4(yr + col);
      c[it][0] = y4.x; c[it][1] = y4.y; c[it][2] = y4.z; c[it][3] = y4.w;
      if (gr) {
        const float4 g4 = ld4(gr + col);
        float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gb) b4 = ld4(gb + col);
        c[it][0] *= sigm<T>(g4.x + b4.x); c[it][1] *= sigm<T>(g4.y + b4.y); c[it][2] *= sigm<T>(g4.z + b4.z); c[it][3] *= sigm<T>(g4.w + b4.w);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) su = fmaf(c[it][k], c[it][k], su);
    }
  }
  float mul = 1.f;
  if (yr && p.post_norm) {
    su = block_sum(su, red);
    mul = p.post_gain / sqrtf(su / (float)D + p.eps);
  }
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    const int col = c0 + it * step;
    if (col < D) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!p.replace) v = ld4(xr + col);
      v.x = fmaf(c[it][0], mul, v.x); v.y = fmaf(c[it][1], mul, v.y); v.z = fmaf(c[it][2], mul, v.z); v.w = fmaf(c[it][3], mul, v.w);
      if (ra) { const float4 a4 = ld4(ra + col); v.x += a4.x; v.y += a4.y; v.z += a4.z; v.w += a4.w; }
      if (write_back) st4(xr + col, v);
      c[it][0] = v.x; c[it][1] = v.y; c[it][2] = v.z; c[it][3] = v.w;
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
  }
  if (!p.out) return;
  T* orow = (T*)p.out + r * p.ldo;
  float g = 1.f;
  if (!p.concat) {
    ss = block_sum(ss, red);
    g = p.gain / sqrtf(ss / (float)D + p.eps);
  }
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    const int col = c0 + it * step;
    if (col < D) st4(orow + col, make_float4(c[it][0] * g, c[it][1] * g, c[it][2] * g, c[it][3] * g));
  }
  const float* cr = p.concat ? p.cat + srow * D : nullptr;
  for (int col = D + c0; col < p.ldo; col += step) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cr && col < 2 * D) v = ld4(cr + col - D);
    st4(orow + col, v);
  }
}

template <typename T>
__device__ __forceinline__ float act_value(float z, int act) {
  if (act == 0) {                         // tanh form of gelu: 0.5 z (1 + tanh(a)) = z sigmoid(2a)
    const float a = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    if (sizeof(T) == 4) return 0.5f * z * (1.f + tanhf(a));
    return z * sigm<T>(2.f * a);
  }
  if (act == 2) return 0.5f * z * (1.f + erff(z * 0.7071067811865476f));     // erf form of gelu
  return z * sigm<T>(z);                   // silu
}

// out[r, c] = act(g[r, c]) * u[r, c] * w(r, c) for c < F, zero for F <= c < ldo (u == nullptr: no second factor);
// w = group_w[r * ldw + c / group] for c < n_groups * group, after them group_w[r * ldw + n_groups] with tail_w, else 1.
// grid (rows, column chunks): few rows (a decoding step) still fill the GPU.  VEC: 4 columns per thread (F, group, strides multiples of 4).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) glu_act_kernel(const T* __restrict__ g, const T* __restrict__ u, int64_t ld, T* __restrict__ out, int64_t ldo,
                                                      int F, int act, const float* __restrict__ group_w, int64_t ldw, int group, int n_groups, int tail_w) {
  const int64_t r = blockIdx.x;
  const T* gr = g + r * ld; const T* ur = u ? u + r * ld : nullptr;
  T* orow = out + r * ldo;
  const float* wr = group_w ? group_w + r * ldw : nullptr;
  constexpr int VW = VEC ? 4 : 1;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VW;
  if (c >= ldo) return;
  float v[VW];
#pragma unroll
  for (int k = 0; k < VW; ++k) v[k] = 0.f;
  if (c < F) {
    float wt = 1.f;
    if (wr) { const int e = c / group; if (e < n_groups) wt = wr[e]; else if (tail_w) wt = wr[n_groups]; }
    if (wt != 0.f) {
      if (VEC) {
        const float4 g4 = ld4(gr + c), u4 = ur ? ld4(ur + c) : make_float4(1.f, 1.f, 1.f, 1.f);
        v[0] = act_value<T>(g4.x, act) * u4.x * wt; v[1] = act_value<T>(g4.y, act) * u4.y * wt;
        v[2] = act_value<T>(g4.z, act) * u4.z * wt; v[3] = act_value<T>(g4.w, act) * u4.w * wt;
      } else {
        v[0] = act_value<T>(ldf(gr + c), act) * (ur ? ldf(ur + c) : 1.f) * wt;
      }
    }
  }
  if (VEC) st4(orow + c, make_float4(v[0], v[1], v[2], v[3]));
  else stf(orow + c, v[0]);
}

}  // namespace

extern "C" int evo_embed_pair_f32(const void* ids, int ids_are_i64, const void* table, const void* pair, float* out, int64_t* prev_state,
                                  int B, int64_t L, int D, int vocab, float scale, int64_t buckets, int64_t mul_prev, int64_t mul_cur, void* stream) {
  EVO_REQUIRE(ids && table && pair && out && D > 0 && vocab > 0 && buckets > 0, "evo_embed_pair_f32: bad arguments");
  if ((int64_t)B * L == 0) return 0;
  dim3 grid((unsigned)((int64_t)B * L)), block(128);
  cudaStream_t st = (cudaStream_t)stream;
  if (ids_are_i64) embed_pair_kernel<long long><<<grid, block, 0, st>>>((const long long*)ids, (const bf16*)table, (const bf16*)pair, out, (long long*)prev_state, L, D, vocab, scale, buckets, mul_prev, mul_cur);
  else embed_pair_kernel<int><<<grid, block, 0, st>>>((const int*)ids, (const bf16*)table, (const bf16*)pair, out, (long long*)prev_state, L, D, vocab, scale, buckets, mul_prev, mul_cur);
  return check_launch("evo_embed_pair_f32");
}

extern "C" int evo_branch_norm(const evo_branch_norm_params* p, void* stream) {
  EVO_REQUIRE(p->x && p->D > 0 && p->rows >= 0, "evo_branch_norm: bad arguments");
  EVO_REQUIRE(p->out == nullptr || p->ldo >= (p->concat ? 2 * p->D : p->D), "evo_branch_norm: ldo too small");
  EVO_REQUIRE(p->y == nullptr || p->ldy >= p->D, "evo_branch_norm: ldy < D");
  EVO_REQUIRE(!p->concat || p->cat, "evo_branch_norm: concat without a second stream");
  EVO_REQUIRE(!p->replace || p->y, "evo_branch_norm: replace without a branch output");
  if (p->rows == 0) return 0;
  dim3 grid((unsigned)p->rows), block(p->D >= 1024 ? 256 : 128);
  const int av = p->dtype ? 16 : 8;          // bytes of 4 activations
  const bool vec = p->D % 4 == 0 && p->ldy % 4 == 0 && p->ldg % 4 == 0 && p->ldo % 4 == 0 && aligned16(p->x) && aligned_to(p->y, av) && aligned_to(p->gate, av) &&
                   aligned_to(p->out, av) && aligned16(p->cat) && aligned_to(p->gate_bias, 8) && aligned_to(p->row_add, 8);
  cudaStream_t st = (cudaStream_t)stream;
  // few rows (a decoding step): the row stays in registers -- one read, one sigmoid per element, a short dependency chain; many rows run
  // faster through the three-pass kernel (fewer registers, more rows in flight per SM; its re-reads hit L1)
  if (vec && p->D <= 16 * (int)block.x && p->rows < 4096) {
    if (p->dtype) branch_norm_cached_kernel<float><<<grid, block, 0, st>>>(*p); else branch_norm_cached_kernel<bf16><<<grid, block, 0, st>>>(*p);
    return check_launch("evo_branch_norm");
  }
  if (p->dtype) { if (vec) branch_norm_kernel<float, true><<<grid, block, 0, st>>>(*p); else branch_norm_kernel<float, false><<<grid, block, 0, st>>>(*p); }
  else { if (vec) branch_norm_kernel<bf16, true><<<grid, block, 0, st>>>(*p); else branch_norm_kernel<bf16, false><<<grid, block, 0, st>>>(*p); }
  return check_launch("evo_branch_norm");
}

extern "C" int evo_glu_act(const void* gate, const void* up, int64_t ld, void* out, int64_t ldo, int64_t rows, int F, int act,
                           const float* group_w, int64_t ldw, int group, int n_groups, int tail_w, int dtype, void* stream) {
  EVO_REQUIRE(gate && out && F > 0 && ldo >= F && act >= 0 && act <= 2, "evo_glu_act: bad arguments");
  EVO_REQUIRE(group_w == nullptr || (group > 0 && n_groups > 0 && ldw >= n_groups + (tail_w ? 1 : 0)), "evo_glu_act: bad groups");
  if (rows == 0) return 0;
  const int av = dtype ? 16 : 8;
  const bool vec = F % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && (group_w == nullptr || (group % 4 == 0)) && aligned_to(gate, av) && aligned_to(up, av) && aligned_to(out, av);
  const int per = 256 * (vec ? 4 : 1);
  EVO_REQUIRE((ldo + per - 1) / per <= 65535, "evo_glu_act: row too wide");
  dim3 grid((unsigned)rows, (unsigned)((ldo + per - 1) / per)), block(256);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype) {
    if (vec) glu_act_kernel<float, true><<<grid, block, 0, st>>>((const float*)gate, (const float*)up, ld, (float*)out, ldo, F, act, group_w, ldw, group, n_groups, tail_w);
    else glu_act_kernel<float, false><<<grid, block, 0, st>>>((const float*)gate, (const float*)up, ld, (float*)out, ldo, F, act, group_w, ldw, group, n_groups, tail_w);
  } else {
    if (vec) glu_act_kernel<bf16, true><<<grid, block, 0, st>>>((const bf16*)gate, (const bf16*)up, ld, (bf16*)out, ldo, F, act, group_w, ldw, group, n_groups, tail_w);
    else glu_act_kernel<bf16, false><<<grid, block, 0, st>>>((const bf16*)gate, (const bf16*)up, ld, (bf16*)out, ldo, F, act, group_w, ldw, group, n_groups, tail_w);
  }
  return check_launch("evo_glu_act");
}

extern "C" int evo_scale_logits(const void* in, int64_t ldi, float* out, int64_t rows, int V, float mul, int dtype, void* stream) {
  EVO_REQUIRE(in && out && V > 0 && ldi >= V, "evo_scale_logits: bad arguments");
  if (rows == 0) return 0;
  const int64_t n = rows * V;
  dim3 grid((unsigned)((n + 255) / 256)), block(256);
  if (dtype) softcap_kernel<float><<<grid, block, 0, (cudaStream_t)stream>>>((const float*)in, ldi, out, rows, V, 0.f, mul);
  else softcap_kernel<bf16><<<grid, block, 0, (cudaStream_t)stream>>>((const bf16*)in, ldi, out, rows, V, 0.f, mul);
  return check_launch("evo_scale_logits");
}
