// Row kernel of designs that norm every sublayer's OUTPUT before it joins the fp32 stream and hand on a learned mix of all
// earlier layers' results (evo_post_norm):
//   t = sum_b scale_b y_b;   x <- x + ln(t) * w + b;   [stack[n-1] <- x;  x <- sum_{j<n} a_j stack[j]];   out <- x  or  ln(x) * w' + b'
// with ln(u) = (u - mean u) / sqrt(mean (u - mean u)^2 + eps).  One CTA per row; the row lives in shared memory between the passes, every
// thread owns the same columns in all of them, and sums, means, variances, the stream and the mix are fp32 whatever the activation type.
#include "common.cuh"
#include "../../include/evo_b200.h"
#include <math.h>
#include <stdint.h>

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// VW consecutive elements as floats, and back (VW = 4: 16 bytes of fp32, 8 of bf16; VW = 1: one element)
template <typename T, int VW> struct Vec;
template <typename T> struct Vec<T, 1> {
  static __device__ __forceinline__ void load(const T* p, float* o) { o[0] = ldf(p); }
  static __device__ __forceinline__ void store(T* p, const float* v) { stf(p, v[0]); }
};
template <> struct Vec<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* o) { const float4 u = *reinterpret_cast<const float4*>(p); o[0] = u.x; o[1] = u.y; o[2] = u.z; o[3] = u.w; }
  static __device__ __forceinline__ void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec<bf16, 4> {
  static __device__ __forceinline__ void load(const bf16* p, float* o) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xffff0000u); o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(bf16* p, const float* v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u; u.x = *reinterpret_cast<const uint32_t*>(&a); u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

// sum over the CTA (blockDim.x a multiple of 32); every thread gets the result; red: 33 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// mean and reciprocal standard deviation of the staged row (this thread's columns: c = tid * VW + k * nt * VW)
template <int VW>
__device__ __forceinline__ void row_moments(const float* xs, int D, float eps, float* red, float& mean, float& rstd) {
  const int tid = threadIdx.x, nt = blockDim.x;
  float s = 0.f;
  for (int c = tid * VW; c < D; c += nt * VW)
#pragma unroll
    for (int u = 0; u < VW; ++u) s += xs[c + u];
  mean = block_sum(s, red) / (float)D;
  float q = 0.f;
  for (int c = tid * VW; c < D; c += nt * VW)
#pragma unroll
    for (int u = 0; u < VW; ++u) { const float d = xs[c + u] - mean; q = fmaf(d, d, q); }
  rstd = 1.0f / sqrtf(block_sum(q, red) / (float)D + eps);
}

template <typename T, int VW>
__global__ void __launch_bounds__(256) post_norm_kernel(evo_post_norm_params p) {
  extern __shared__ __align__(16) float xs[];          // [D rounded up to 4] + 33
  const int D = p.D, tid = threadIdx.x, nt = blockDim.x;
  float* red = xs + (D + 3) / 4 * 4;
  const int64_t r = blockIdx.x;
  const int64_t src = p.gather ? p.gather[r] : r;
  const float* xin = (p.x_in ? p.x_in : p.x) + src * D;
  if (p.n_in > 0) {
    for (int c = tid * VW; c < D; c += nt * VW) {
      float t[VW];
#pragma unroll
      for (int u = 0; u < VW; ++u) t[u] = 0.f;
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        if (b < p.n_in) {
          float y[VW];
          Vec<T, VW>::load((const T*)p.y[b] + src * p.ldy[b] + c, y);
#pragma unroll
          for (int u = 0; u < VW; ++u) t[u] = fmaf(p.scale[b], y[u], t[u]);
        }
      }
      Vec<float, VW>::store(xs + c, t);
    }
    float mean, rstd;
    row_moments<VW>(xs, D, p.eps, red, mean, rstd);
    for (int c = tid * VW; c < D; c += nt * VW) {
      float t[VW], x[VW], w[VW], b[VW];
      Vec<float, VW>::load(xs + c, t);
      Vec<float, VW>::load(xin + c, x);
      Vec<bf16, VW>::load((const bf16*)p.norm_w + c, w);
      Vec<bf16, VW>::load((const bf16*)p.norm_b + c, b);
#pragma unroll
      for (int u = 0; u < VW; ++u) t[u] = x[u] + (fmaf((t[u] - mean) * rstd, w[u], b[u]));
      Vec<float, VW>::store(xs + c, t);
    }
  } else {
    for (int c = tid * VW; c < D; c += nt * VW) {
      float x[VW];
      Vec<float, VW>::load(xin + c, x);
      Vec<float, VW>::store(xs + c, x);
    }
  }
  if (p.mix_n > 0) {
    const bf16* mw = (const bf16*)p.mix_w;
    const int last = p.mix_n - 1;
    const float wl = __bfloat162float(mw[last]);
    for (int c = tid * VW; c < D; c += nt * VW) {
      float x[VW], acc[VW];
      Vec<float, VW>::load(xs + c, x);
      if (!p.gather) Vec<float, VW>::store(p.stack + last * p.stack_stride + src * D + c, x);
#pragma unroll
      for (int u = 0; u < VW; ++u) acc[u] = 0.f;
      for (int j = 0; j < last; ++j) {
        float e[VW];
        Vec<float, VW>::load(p.stack + j * p.stack_stride + src * D + c, e);
        const float wj = __bfloat162float(mw[j]);
#pragma unroll
        for (int u = 0; u < VW; ++u) acc[u] = fmaf(wj, e[u], acc[u]);
      }
#pragma unroll
      for (int u = 0; u < VW; ++u) acc[u] = fmaf(wl, x[u], acc[u]);
      Vec<float, VW>::store(xs + c, acc);
    }
  }
  if (!p.gather && (p.n_in > 0 || p.mix_n > 0 || (p.x_in && p.x_in != p.x))) {
    float* xo = p.x + src * D;
    for (int c = tid * VW; c < D; c += nt * VW) {
      float x[VW];
      Vec<float, VW>::load(xs + c, x);
      Vec<float, VW>::store(xo + c, x);
    }
  }
  if (!p.out) return;
  float mean = 0.f, rstd = 1.f;
  if (p.out_norm_w) row_moments<VW>(xs, D, p.eps, red, mean, rstd);
  T* o = (T*)p.out + r * p.ldo;
  for (int c = tid * VW; c < p.ldo; c += nt * VW) {
    float v[VW];
#pragma unroll
    for (int u = 0; u < VW; ++u) v[u] = 0.f;
    if (c < D) {                             // VW == 4 only with D % 4 == 0: a group lies inside the row or in the padding
      Vec<float, VW>::load(xs + c, v);
      if (p.out_norm_w) {
        float w[VW], b[VW];
        Vec<bf16, VW>::load((const bf16*)p.out_norm_w + c, w);
        Vec<bf16, VW>::load((const bf16*)p.out_norm_b + c, b);
#pragma unroll
        for (int u = 0; u < VW; ++u) v[u] = fmaf((v[u] - mean) * rstd, w[u], b[u]);
      }
    }
    Vec<T, VW>::store(o + c, v);
  }
}

inline bool al(const void* p, int n) { return ((uintptr_t)p & (uintptr_t)(n - 1)) == 0; }

}  // namespace

extern "C" int evo_post_norm(const evo_post_norm_params* p, void* stream) {
  EVO_REQUIRE(p->x && p->D > 0 && p->rows >= 0 && p->n_in >= 0 && p->n_in <= 2, "evo_post_norm: bad arguments");
  for (int b = 0; b < p->n_in; ++b) EVO_REQUIRE(p->y[b] && p->ldy[b] >= p->D, "evo_post_norm: input %d missing or too narrow", b);
  EVO_REQUIRE(p->n_in == 0 || (p->norm_w && p->norm_b), "evo_post_norm: the norm of the inputs needs weight and bias");
  EVO_REQUIRE(p->mix_n == 0 || (p->mix_n > 0 && p->stack && p->mix_w && p->stack_stride >= p->rows * (int64_t)p->D), "evo_post_norm: bad mix");
  EVO_REQUIRE(!p->out || p->ldo >= p->D, "evo_post_norm: ldo too small");
  EVO_REQUIRE(!p->out_norm_w || p->out_norm_b, "evo_post_norm: the output norm needs weight and bias");
  if (p->rows == 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)(p->D + 3) / 4 * 4 + 33);
  EVO_REQUIRE(smem <= 200 * 1024, "evo_post_norm: width %d too large for one CTA's shared memory", p->D);
  const int av = p->dtype ? 16 : 8;          // bytes of 4 activations
  bool vec = p->D % 4 == 0 && (!p->out || p->ldo % 4 == 0) && al(p->x, 16) && al(p->x_in, 16) && al(p->out, av) && al(p->norm_w, 8) && al(p->norm_b, 8) &&
             al(p->out_norm_w, 8) && al(p->out_norm_b, 8) && al(p->stack, 16) && p->stack_stride % 4 == 0;
  for (int b = 0; b < p->n_in; ++b) vec = vec && al(p->y[b], av) && p->ldy[b] % 4 == 0;
  auto kern = p->dtype ? (vec ? post_norm_kernel<float, 4> : post_norm_kernel<float, 1>) : (vec ? post_norm_kernel<bf16, 4> : post_norm_kernel<bf16, 1>);
  if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int threads = p->D >= 2048 ? 256 : 128;
  kern<<<(unsigned)p->rows, threads, smem, (cudaStream_t)stream>>>(*p);
  return check_launch("evo_post_norm");
}
