// Row kernels of designs whose layers run several branches side by side on norms of the same fp32 stream:
//   evo_sum_norm          x += sum of (optionally RMS-normed) branch outputs, then one or two norms of the new x
//   evo_conv_act          short causal convolution per channel on columns of a projection, with carried inputs, then SiLU
//   evo_xielu             the xIELU activation between the two feed-forward products
//   evo_gated_group_norm  y * silu(gate), RMS norm in equal parts of the row, weight
// Sums of squares, norms and the stream are fp32 whatever the activation type.
#include "common.cuh"
#include "../../include/evo_b200.h"
#include <math.h>
#include <algorithm>
#include <stdint.h>

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// four consecutive elements (16 bytes of fp32, 8 of bf16) as floats, and back
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float* o) { const float4 u = *reinterpret_cast<const float4*>(p); o[0] = u.x; o[1] = u.y; o[2] = u.z; o[3] = u.w; }
  static __device__ __forceinline__ void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec4<bf16> {
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
template <typename T> inline bool aligned4(const void* p) { return ((uintptr_t)p & (4 * sizeof(T) - 1)) == 0; }

// sum over the CTA (blockDim.x a multiple of 32, at most 1024); every thread gets the result; red: 33 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();                       // red may still be read from the previous sum
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

// ---- evo_sum_norm: one CTA per row; the new row of x is kept in shared memory between the passes
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) sum_norm_kernel(evo_sum_norm_params p) {
  extern __shared__ float xs[];          // [D] + 33
  float* red = xs + p.D;
  const int64_t r = blockIdx.x;
  const int64_t src = p.gather ? p.gather[r] : r;
  const int D = p.D, tid = threadIdx.x, nt = blockDim.x;
  float rstd[EVO_SUM_NORM_BRANCHES];
#pragma unroll
  for (int b = 0; b < EVO_SUM_NORM_BRANCHES; ++b) {
    rstd[b] = 1.f;
    if (b < p.n_branches && p.norm_w[b]) {
      const T* y = (const T*)p.y[b] + src * p.ldy[b];
      float ss = 0.f;
      if (VEC) {
        for (int c = tid * 4; c < D; c += nt * 4) { float v[4]; Vec4<T>::load(y + c, v); ss = fmaf(v[0], v[0], fmaf(v[1], v[1], fmaf(v[2], v[2], fmaf(v[3], v[3], ss)))); }
      } else {
        for (int c = tid; c < D; c += nt) { const float v = ldf(y + c); ss = fmaf(v, v, ss); }
      }
      rstd[b] = 1.0f / sqrtf(block_sum(ss, red) / (float)D + p.eps);
    }
  }
  float* xr = p.x + src * D;
  float ss = 0.f;
  if (VEC) {
    for (int c = tid * 4; c < D; c += nt * 4) {
      float v[4], add[4] = {0.f, 0.f, 0.f, 0.f};
      Vec4<float>::load(xr + c, v);
#pragma unroll
      for (int b = 0; b < EVO_SUM_NORM_BRANCHES; ++b) {
        if (b < p.n_branches) {
          float y[4];
          Vec4<T>::load((const T*)p.y[b] + src * p.ldy[b] + c, y);
          if (p.norm_w[b]) {
            float w[4];
            Vec4<bf16>::load((const bf16*)p.norm_w[b] + c, w);
#pragma unroll
            for (int u = 0; u < 4; ++u) y[u] = y[u] * rstd[b] * w[u];
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) add[u] = fmaf(p.scale[b], y[u], add[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) { v[u] += add[u]; ss = fmaf(v[u], v[u], ss); }
      Vec4<float>::store(xs + c, v);
      if (p.n_branches > 0 && !p.gather) Vec4<float>::store(xr + c, v);
    }
  } else
  for (int c = tid; c < D; c += nt) {
    float v = xr[c];
    float add = 0.f;
#pragma unroll
    for (int b = 0; b < EVO_SUM_NORM_BRANCHES; ++b) {
      if (b < p.n_branches) {
        float y = ldf((const T*)p.y[b] + src * p.ldy[b] + c);
        if (p.norm_w[b]) y = y * rstd[b] * __bfloat162float(((const bf16*)p.norm_w[b])[c]);
        add = fmaf(p.scale[b], y, add);
      }
    }
    v += add;
    xs[c] = v;
    if (p.n_branches > 0 && !p.gather) xr[c] = v;
    ss = fmaf(v, v, ss);
  }
  if (!p.out[0] && !p.out[1]) return;
  const float rs = 1.0f / sqrtf(block_sum(ss, red) / (float)D + p.eps);
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    if (!p.out[n]) continue;
    T* o = (T*)p.out[n] + r * p.ldo;
    const bf16* w = (const bf16*)p.w[n];
    if (VEC) {
      for (int c = tid * 4; c < p.ldo; c += nt * 4) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (c < D) {                     // D % 4 == 0: a group of four lies inside the row or in the padding
          float wv[4];
          Vec4<bf16>::load(w + c, wv);
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = xs[c + u] * rs * wv[u];
        }
        Vec4<T>::store(o + c, v);
      }
    } else
    for (int c = tid; c < p.ldo; c += nt) stf(o + c, c < D ? xs[c] * rs * __bfloat162float(w[c]) : 0.f);
  }
}

// ---- evo_conv_act: a thread owns one channel of one sequence over RT consecutive rows, its last taps inputs in registers
constexpr int CONV_RT = 32, CONV_MAX_TAPS = 8;

// four channels per thread (8- or 16-byte accesses), taps known at compile time
template <typename T, int TAPS>
__global__ void __launch_bounds__(128) conv_act4_kernel(evo_conv_act_params p, int write_carry) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= p.C) return;
  constexpr int HALO = TAPS - 1;
  const int b = blockIdx.z;
  const int64_t t0 = (int64_t)blockIdx.y * CONV_RT, t1 = min(p.L, t0 + CONV_RT);
  const T* in = (const T*)p.in + (int64_t)b * p.L * p.ld + c;
  float* carry = p.carry ? p.carry + (int64_t)b * HALO * p.C + c : nullptr;
  float w[4][TAPS], win[HALO > 0 ? HALO : 1][4], bias[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int j = 0; j < TAPS; ++j) w[u][j] = __bfloat162float(((const bf16*)p.weight)[(int64_t)(c + u) * TAPS + j]);
  if (p.bias) Vec4<bf16>::load((const bf16*)p.bias + c, bias);
#pragma unroll
  for (int j = 0; j < HALO; ++j) {
    const int64_t s = t0 - HALO + j;
    win[j][0] = win[j][1] = win[j][2] = win[j][3] = 0.f;
    if (s >= 0) Vec4<T>::load(in + s * p.ld, win[j]);
    else if (carry && !p.zero_start) Vec4<float>::load(carry + (int64_t)(HALO + s) * p.C, win[j]);
  }
  for (int64_t t = t0; t < t1; ++t) {
    float cur[4], acc[4];
    Vec4<T>::load(in + t * p.ld, cur);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float a = fmaf(w[u][HALO], cur[u], bias[u]);
#pragma unroll
      for (int j = 0; j < HALO; ++j) a = fmaf(w[u][j], win[j][u], a);
      acc[u] = p.act == 1 ? silu_f(a) : a;
    }
    Vec4<T>::store((T*)p.out + ((int64_t)b * p.L + t) * p.ldo + c, acc);
#pragma unroll
    for (int j = 0; j + 1 < HALO; ++j)
#pragma unroll
      for (int u = 0; u < 4; ++u) win[j][u] = win[j + 1][u];
    if (HALO > 0) {
#pragma unroll
      for (int u = 0; u < 4; ++u) win[HALO - 1][u] = cur[u];
    }
  }
  if (write_carry && carry && t1 == p.L) {
#pragma unroll
    for (int j = 0; j < HALO; ++j) Vec4<float>::store(carry + (int64_t)j * p.C, win[j]);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) conv_act_kernel(evo_conv_act_params p, int write_carry) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int b = blockIdx.z, taps = p.taps, halo = taps - 1;
  const int64_t t0 = (int64_t)blockIdx.y * CONV_RT, t1 = min(p.L, t0 + CONV_RT);
  const T* in = (const T*)p.in + (int64_t)b * p.L * p.ld + c;
  float* carry = p.carry ? p.carry + (int64_t)b * halo * p.C + c : nullptr;
  float w[CONV_MAX_TAPS], win[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = j < taps ? __bfloat162float(((const bf16*)p.weight)[(int64_t)c * taps + j]) : 0.f;
  const float bias = p.bias ? __bfloat162float(((const bf16*)p.bias)[c]) : 0.f;
  // win[j] = input at t - halo + j for the row t about to be computed; filled for j < halo here, win[halo] in the loop
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
    win[j] = 0.f;
    if (j < halo) {
      const int64_t s = t0 - halo + j;
      if (s >= 0) win[j] = ldf(in + s * p.ld);
      else if (carry && !p.zero_start) win[j] = carry[(int64_t)(halo + s) * p.C];
    }
  }
  win[CONV_MAX_TAPS - 1] = 0.f;
  for (int64_t t = t0; t < t1; ++t) {
    const float cur = ldf(in + t * p.ld);
    float acc = bias;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      if (j < halo) acc = fmaf(w[j], win[j], acc);
      else if (j == halo) acc = fmaf(w[j], cur, acc);
    }
    if (p.act == 1) acc = silu_f(acc);
    stf((T*)p.out + ((int64_t)b * p.L + t) * p.ldo + c, acc);
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
      if (j + 1 < halo) win[j] = win[j + 1];
      else if (j + 1 == halo) win[j] = cur;
    }
  }
  // after the last row win[0 .. halo) holds the last halo inputs (carried ones included when L < halo)
  if (write_carry && carry && t1 == p.L) {
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
      if (j < halo) carry[(int64_t)j * p.C] = win[j];
  }
}

// the carried inputs of a call whose rows were spread over several threads per channel: written after every row has been read
template <typename T>
__global__ void __launch_bounds__(128) conv_carry_kernel(evo_conv_act_params p) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const int b = blockIdx.z, halo = p.taps - 1;
  const T* in = (const T*)p.in + (int64_t)b * p.L * p.ld + c;
  float* carry = p.carry + (int64_t)b * halo * p.C + c;
  float keep[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
    keep[j] = 0.f;
    if (j < halo) {
      const int64_t s = p.L - halo + j;
      if (s >= 0) keep[j] = ldf(in + s * p.ld);
      else if (!p.zero_start) keep[j] = carry[(int64_t)(halo + s) * p.C];
    }
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
    if (j < halo) carry[(int64_t)j * p.C] = keep[j];
}

// ---- evo_xielu
template <typename T>
__global__ void __launch_bounds__(256) xielu_kernel(const T* __restrict__ z, int64_t ldz, const bf16* __restrict__ coef, T* __restrict__ out, int64_t ldo,
                                                    int64_t rows, int F) {
  const float pa = __bfloat162float(coef[0]), qa = __bfloat162float(coef[1]);
  // softplus in the form that neither overflows nor loses small values
  const float ap = fmaxf(pa, 0.f) + log1pf(expf(-fabsf(pa)));
  const float an = 0.5f + fmaxf(qa, 0.f) + log1pf(expf(-fabsf(qa)));
  const int64_t total = rows * ldo;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / ldo; const int c = (int)(i - r * ldo);
    float o = 0.f;
    if (c < F) {
      const float v = ldf(z + r * ldz + c);
      o = v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v);
    }
    stf(out + i, o);
  }
}

// four columns per thread, rows along grid.y: no division per element
template <typename T>
__global__ void __launch_bounds__(256) xielu4_kernel(const T* __restrict__ z, int64_t ldz, const bf16* __restrict__ coef, T* __restrict__ out, int64_t ldo,
                                                     int64_t rows, int F) {
  const float pa = __bfloat162float(coef[0]), qa = __bfloat162float(coef[1]);
  const float ap = fmaxf(pa, 0.f) + log1pf(expf(-fabsf(pa)));
  const float an = 0.5f + fmaxf(qa, 0.f) + log1pf(expf(-fabsf(qa)));
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= ldo) return;
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
    float v[4] = {0.f, 0.f, 0.f, 0.f}, o[4];
    if (c < F) Vec4<T>::load(z + r * ldz + c, v);           // ldz >= F rounded up to four: the group may read pad columns of z, masked below
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float x = v[u];
      // bf16 activations: e^x - 1 from the fast exponential (its absolute error is far below the output's rounding step)
      const float em1 = sizeof(T) == 2 ? __expf(x) - 1.f : expm1f(x);
      o[u] = c + u < F ? (x > 0.f ? fmaf(ap * x, x, 0.5f * x) : fmaf(an, em1 - x, 0.5f * x)) : 0.f;
    }
    Vec4<T>::store(out + r * ldo + c, o);
  }
}

// ---- evo_gated_group_norm: one warp per (row, part)
// the same with four entries per access (part size, strides and bases multiples of four entries)
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm4_kernel(const float* __restrict__ y, const T* __restrict__ gate, int64_t ldg, const bf16* __restrict__ nw,
                                                                T* __restrict__ out, int64_t ldo, int64_t rows, int width, int groups, float eps) {
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= rows * groups) return;
  const int64_t r = wid / groups; const int g = (int)(wid % groups);
  const int gs = width / groups, c0 = g * gs;
  const float* yr = y + r * width + c0;
  const T* gr = gate + r * ldg + c0;
  float ss = 0.f;
  for (int c = lane * 4; c < gs; c += 128) {
    float a[4], b[4];
    Vec4<float>::load(yr + c, a); Vec4<T>::load(gr + c, b);
#pragma unroll
    for (int u = 0; u < 4; ++u) { const float v = a[u] * silu_f(b[u]); ss = fmaf(v, v, ss); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rs = 1.0f / sqrtf(ss / (float)gs + eps);
  T* orow = out + r * ldo;
  for (int c = lane * 4; c < gs; c += 128) {
    float a[4], b[4], w[4];
    Vec4<float>::load(yr + c, a); Vec4<T>::load(gr + c, b); Vec4<bf16>::load(nw + c0 + c, w);
#pragma unroll
    for (int u = 0; u < 4; ++u) a[u] = a[u] * silu_f(b[u]) * rs * w[u];
    Vec4<T>::store(orow + c0 + c, a);
  }
  if (g == groups - 1)
    for (int64_t c = width + lane; c < ldo; c += 32) stf(orow + c, 0.f);
}

template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int64_t ldg, const bf16* __restrict__ nw,
                                                               T* __restrict__ out, int64_t ldo, int64_t rows, int width, int groups, float eps) {
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= rows * groups) return;
  const int64_t r = wid / groups; const int g = (int)(wid % groups);
  const int gs = width / groups, c0 = g * gs;
  const float* yr = y + r * width + c0;
  const T* gr = gate + r * ldg + c0;
  float ss = 0.f;
  for (int c = lane; c < gs; c += 32) { const float v = yr[c] * silu_f(ldf(gr + c)); ss = fmaf(v, v, ss); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rs = 1.0f / sqrtf(ss / (float)gs + eps);
  T* orow = out + r * ldo;
  for (int c = lane; c < gs; c += 32) stf(orow + c0 + c, yr[c] * silu_f(ldf(gr + c)) * rs * __bfloat162float(nw[c0 + c]));
  if (g == groups - 1)
    for (int64_t c = width + lane; c < ldo; c += 32) stf(orow + c, 0.f);
}

}  // namespace

extern "C" int evo_sum_norm(const evo_sum_norm_params* p, void* stream) {
  EVO_REQUIRE(p->x && p->D > 0 && p->rows >= 0 && p->n_branches >= 0 && p->n_branches <= EVO_SUM_NORM_BRANCHES, "evo_sum_norm: bad arguments");
  for (int b = 0; b < p->n_branches; ++b) EVO_REQUIRE(p->y[b] && p->ldy[b] >= p->D, "evo_sum_norm: branch %d missing or too narrow", b);
  for (int n = 0; n < 2; ++n) EVO_REQUIRE(!p->out[n] || (p->w[n] && p->ldo >= p->D), "evo_sum_norm: output %d without weight or too narrow", n);
  if (p->rows == 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)p->D + 33);
  EVO_REQUIRE(smem <= 200 * 1024, "evo_sum_norm: width %d too large for one CTA's shared memory", p->D);
  cudaStream_t st = (cudaStream_t)stream;
  // four elements per access when every row of every operand starts on a multiple of four elements
  bool vec = p->D % 4 == 0 && p->ldo % 4 == 0 && ((uintptr_t)p->x & 15) == 0;
  for (int b = 0; b < p->n_branches; ++b) {
    vec = vec && p->ldy[b] % 4 == 0 && (p->dtype ? aligned4<float>(p->y[b]) : aligned4<bf16>(p->y[b]));
    if (p->norm_w[b]) vec = vec && aligned4<bf16>(p->norm_w[b]);
  }
  for (int n = 0; n < 2; ++n)
    if (p->out[n]) vec = vec && aligned4<bf16>(p->w[n]) && (p->dtype ? aligned4<float>(p->out[n]) : aligned4<bf16>(p->out[n]));
  auto kern = p->dtype ? (vec ? sum_norm_kernel<float, true> : sum_norm_kernel<float, false>) : (vec ? sum_norm_kernel<bf16, true> : sum_norm_kernel<bf16, false>);
  if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)p->rows, 256, smem, st>>>(*p);
  return check_launch("evo_sum_norm");
}

extern "C" int evo_conv_act(const evo_conv_act_params* p, void* stream) {
  EVO_REQUIRE(p->in && p->weight && p->out && p->C > 0 && p->taps >= 1 && p->taps <= CONV_MAX_TAPS, "evo_conv_act: bad arguments (taps 1..%d)", CONV_MAX_TAPS);
  EVO_REQUIRE(p->ld >= p->C && p->ldo >= p->C && p->B >= 0 && p->L >= 0, "evo_conv_act: bad shape");
  if (p->B == 0 || p->L == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned chunks = (unsigned)((p->L + CONV_RT - 1) / CONV_RT);
  const dim3 grid((p->C + 127) / 128, chunks, p->B);
  // with one thread per (sequence, channel) that thread reads the carried inputs before it replaces them; otherwise a second launch does
  const int own = chunks == 1;
  const bool vec = p->C % 4 == 0 && p->ld % 4 == 0 && p->ldo % 4 == 0 && p->taps <= 4 && (!p->carry || ((uintptr_t)p->carry & 15) == 0) &&
                   (!p->bias || aligned4<bf16>(p->bias)) &&
                   (p->dtype ? aligned4<float>(p->in) && aligned4<float>(p->out) : aligned4<bf16>(p->in) && aligned4<bf16>(p->out));
  if (vec) {
    const dim3 g4((p->C / 4 + 127) / 128, chunks, p->B);
#define EVO_CONV4(TT) \
    switch (p->taps) { \
      case 1: conv_act4_kernel<TT, 1><<<g4, 128, 0, st>>>(*p, own); break; \
      case 2: conv_act4_kernel<TT, 2><<<g4, 128, 0, st>>>(*p, own); break; \
      case 3: conv_act4_kernel<TT, 3><<<g4, 128, 0, st>>>(*p, own); break; \
      default: conv_act4_kernel<TT, 4><<<g4, 128, 0, st>>>(*p, own); break; \
    }
    if (p->dtype) { EVO_CONV4(float) } else { EVO_CONV4(bf16) }
#undef EVO_CONV4
  } else if (p->dtype) conv_act_kernel<float><<<grid, 128, 0, st>>>(*p, own); else conv_act_kernel<bf16><<<grid, 128, 0, st>>>(*p, own);
  int rc = check_launch("evo_conv_act");
  if (rc || own || !p->carry || p->taps == 1) return rc;
  const dim3 g2((p->C + 127) / 128, 1, p->B);
  if (p->dtype) conv_carry_kernel<float><<<g2, 128, 0, st>>>(*p); else conv_carry_kernel<bf16><<<g2, 128, 0, st>>>(*p);
  return check_launch("evo_conv_act");
}

extern "C" int evo_xielu(const void* z, int64_t ldz, const void* coef, void* out, int64_t ldo, int64_t rows, int F, int dtype, void* stream) {
  EVO_REQUIRE(z && coef && out && F > 0 && ldz >= F && ldo >= F && rows >= 0, "evo_xielu: bad arguments");
  if (rows == 0) return 0;
  const int64_t total = rows * ldo;
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, (int64_t)device_sm_count() * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (ldz % 4 == 0 && ldo % 4 == 0 && ldz >= (F + 3) / 4 * 4 && (dtype ? aligned4<float>(z) && aligned4<float>(out) : aligned4<bf16>(z) && aligned4<bf16>(out))) {
    // a thread walks several rows of its four columns, so that the two softplus of the coefficients are paid once per many elements
    const dim3 g4((unsigned)((ldo / 4 + 255) / 256), (unsigned)std::min<int64_t>(rows, std::max<int64_t>(1, (int64_t)device_sm_count() * 8 / ((ldo / 4 + 255) / 256))));
    if (dtype) xielu4_kernel<float><<<g4, 256, 0, st>>>((const float*)z, ldz, (const bf16*)coef, (float*)out, ldo, rows, F);
    else xielu4_kernel<bf16><<<g4, 256, 0, st>>>((const bf16*)z, ldz, (const bf16*)coef, (bf16*)out, ldo, rows, F);
    return check_launch("evo_xielu");
  }
  if (dtype) xielu_kernel<float><<<grid, 256, 0, st>>>((const float*)z, ldz, (const bf16*)coef, (float*)out, ldo, rows, F);
  else xielu_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)z, ldz, (const bf16*)coef, (bf16*)out, ldo, rows, F);
  return check_launch("evo_xielu");
}

extern "C" int evo_gated_group_norm(const float* y, const void* gate, int64_t ldg, const void* norm_w, void* out, int64_t ldo,
                                    int64_t rows, int width, int groups, float eps, int dtype, void* stream) {
  EVO_REQUIRE(y && gate && norm_w && out && width > 0 && groups > 0 && width % groups == 0 && ldo >= width && ldg >= width, "evo_gated_group_norm: bad arguments");
  if (rows == 0) return 0;
  const int64_t warps = rows * groups;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((warps + 7) / 8);
  if ((width / groups) % 4 == 0 && ldg % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)y & 15) == 0 && aligned4<bf16>(norm_w) &&
      (dtype ? aligned4<float>(gate) && aligned4<float>(out) : aligned4<bf16>(gate) && aligned4<bf16>(out))) {
    if (dtype) gated_group_norm4_kernel<float><<<grid, 256, 0, st>>>(y, (const float*)gate, ldg, (const bf16*)norm_w, (float*)out, ldo, rows, width, groups, eps);
    else gated_group_norm4_kernel<bf16><<<grid, 256, 0, st>>>(y, (const bf16*)gate, ldg, (const bf16*)norm_w, (bf16*)out, ldo, rows, width, groups, eps);
    return check_launch("evo_gated_group_norm");
  }
  if (dtype) gated_group_norm_kernel<float><<<grid, 256, 0, st>>>(y, (const float*)gate, ldg, (const bf16*)norm_w, (float*)out, ldo, rows, width, groups, eps);
  else gated_group_norm_kernel<bf16><<<grid, 256, 0, st>>>(y, (const bf16*)gate, ldg, (const bf16*)norm_w, (bf16*)out, ldo, rows, width, groups, eps);
  return check_launch("evo_gated_group_norm");
}
