// Preparation of attention inputs whose query and key are normed (over the whole projection, or head by head), rotated in part and, for
// the query, scaled by a temperature that grows with the position (evo_qk_prep), and
// the pooled rows of a key/value cache (evo_pool_rows): the mean of every completed block of consecutive cache rows.
// Biases, sums of squares, norms, angles and rotations are fp32; results are rounded once, when they are stored.
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
template <typename T> inline bool aligned4(const void* p) { return !p || ((uintptr_t)p & (4 * sizeof(T) - 1)) == 0; }

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

// hr[0 .. H) and hr[H .. H + G): what every head's staged query / key entries are multiplied by -- the reciprocal root mean square of the
// whole projection (sq, sk: this thread's part of its sum of squares) or of the head alone, and for the query the position's temperature
__device__ __forceinline__ void head_scales(const evo_qk_prep_params& p, const float* qs, const float* ks, float sq, float sk, float* red, float* hr, int64_t pos) {
  const int qw = p.H * p.dk, kw = p.G * p.dk;
  const float temp = p.q_temp_every > 0 ? 1.f + p.q_temp_coef * logf((float)((pos + 1) / p.q_temp_every) + 1.f) : 1.f;
  if (!p.norm_per_head) {
    const float rq = p.q_norm_w ? 1.0f / sqrtf(block_sum(sq, red) / (float)qw + p.eps) : 1.f;
    const float rk = p.k_norm_w ? 1.0f / sqrtf(block_sum(sk, red) / (float)kw + p.eps) : 1.f;
    for (int i = threadIdx.x; i < p.H + p.G; i += blockDim.x) hr[i] = i < p.H ? rq * temp : rk;
  } else {
    __syncthreads();                                           // the staged rows are complete
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int i = w; i < p.H + p.G; i += nw) {
      const float* src = i < p.H ? qs + i * p.dk : ks + (i - p.H) * p.dk;
      float ss = 0.f;
      for (int e = lane; e < p.dk; e += 32) ss = fmaf(src[e], src[e], ss);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const bool normed = i < p.H ? p.q_norm_w != nullptr : p.k_norm_w != nullptr;
      if (lane == 0) hr[i] = (normed ? 1.0f / sqrtf(ss / (float)p.dk + p.eps) : 1.f) * (i < p.H ? temp : 1.f);
    }
  }
  __syncthreads();
}

// one CTA per row: the biased q and k rows wait in shared memory for their sums of squares, then are normed, turned and stored
template <typename T>
__global__ void __launch_bounds__(256) qk_prep_kernel(evo_qk_prep_params p) {
  extern __shared__ float sm[];
  const int qw = p.H * p.dk, kw = p.G * p.dk, vw = p.G * p.dv;
  float* qs = sm;              // [qw]
  float* ks = qs + qw;         // [kw]
  float* red = ks + kw;        // [33]
  float* hr = red + 33;        // [H + G] reciprocal root mean squares, per head
  const int64_t row = blockIdx.x;
  const int b = (int)(row / p.L);
  const int64_t t = row - (int64_t)b * p.L;
  const int64_t pos = (p.pos_dev ? *p.pos_dev : p.pos0) + t;
  const int tid = threadIdx.x, nt = blockDim.x;
  T* q = (T*)p.q + row * p.ld;
  const T* k = (const T*)p.k + row * p.ld;
  const T* v = (const T*)p.v + row * p.ld;
  T* crow = (T*)p.cache + (int64_t)b * p.cache_batch_stride + pos * p.cache_row;
  const bf16* qb = (const bf16*)p.q_bias; const bf16* kb = (const bf16*)p.k_bias; const bf16* vb = (const bf16*)p.v_bias;
  float sq = 0.f, sk = 0.f;
  for (int c = tid; c < qw; c += nt) { const float x = ldf(q + c) + (qb ? __bfloat162float(qb[c]) : 0.f); qs[c] = x; sq = fmaf(x, x, sq); }
  for (int c = tid; c < kw; c += nt) { const float x = ldf(k + c) + (kb ? __bfloat162float(kb[c]) : 0.f); ks[c] = x; sk = fmaf(x, x, sk); }
  for (int c = tid; c < vw; c += nt) stf(crow + kw + c, ldf(v + c) + (vb ? __bfloat162float(vb[c]) : 0.f));
  head_scales(p, qs, ks, sq, sk, red, hr, pos);
  const bf16* qn = (const bf16*)p.q_norm_w; const bf16* kn = (const bf16*)p.k_norm_w;
  const int half = p.rot_dims / 2;
  // an entry is written by the thread that owns it; a turned pair (e, e + half) is owned by the thread of e
  for (int part = 0; part < 2; ++part) {
    const int width = part == 0 ? qw : kw;
    const float* src = part == 0 ? qs : ks;
    const bf16* nw = part == 0 ? qn : kn;
    const float* hrs = part == 0 ? hr : hr + p.H;
    T* dst = part == 0 ? q : crow;
    for (int c = tid; c < width; c += nt) {
      const int e = c % p.dk, wc = p.norm_per_head ? e : c;       // a per-head norm weight has dk entries
      const float rs = hrs[c / p.dk];
      if (e >= p.rot_dims) { stf(dst + c, src[c] * rs * (nw ? __bfloat162float(nw[wc]) : 1.f)); continue; }
      if (e >= half) continue;
      const float u = src[c] * rs * (nw ? __bfloat162float(nw[wc]) : 1.f);
      const float w = src[c + half] * rs * (nw ? __bfloat162float(nw[wc + half]) : 1.f);
      float sn, cs;
      sincosf((float)pos * p.freq[e], &sn, &cs);
      stf(dst + c, u * cs - w * sn);
      stf(dst + c + half, w * cs + u * sn);
    }
  }
}

// the same with four entries per access (head sizes, rotated halves, strides and bases multiples of four entries); the row's
// sines and cosines are computed once and shared by all heads
template <typename T>
__global__ void __launch_bounds__(256) qk_prep4_kernel(evo_qk_prep_params p) {
  extern __shared__ __align__(16) float sm[];
  const int qw = p.H * p.dk, kw = p.G * p.dk, vw = p.G * p.dv, half = p.rot_dims / 2;
  float* qs = sm;              // [qw]
  float* ks = qs + qw;         // [kw]
  float* cs = ks + kw;         // [half] cosines, then [half] sines
  float* red = cs + 2 * half + (4 - (2 * half) % 4) % 4;      // [33]
  float* hr = red + 33;                                        // [H + G] reciprocal root mean squares, per head
  const int64_t row = blockIdx.x;
  const int b = (int)(row / p.L);
  const int64_t t = row - (int64_t)b * p.L;
  const int64_t pos = (p.pos_dev ? *p.pos_dev : p.pos0) + t;
  const int tid = threadIdx.x, nt = blockDim.x;
  T* q = (T*)p.q + row * p.ld;
  const T* k = (const T*)p.k + row * p.ld;
  const T* v = (const T*)p.v + row * p.ld;
  T* crow = (T*)p.cache + (int64_t)b * p.cache_batch_stride + pos * p.cache_row;
  const bf16* qb = (const bf16*)p.q_bias; const bf16* kb = (const bf16*)p.k_bias; const bf16* vb = (const bf16*)p.v_bias;
  for (int e = tid; e < half; e += nt) sincosf((float)pos * p.freq[e], cs + half + e, cs + e);
  float sq = 0.f, sk = 0.f;
  for (int c = tid * 4; c < qw; c += nt * 4) {
    float x[4], bb[4] = {0.f, 0.f, 0.f, 0.f};
    Vec4<T>::load(q + c, x);
    if (qb) Vec4<bf16>::load(qb + c, bb);
#pragma unroll
    for (int u = 0; u < 4; ++u) { x[u] += bb[u]; sq = fmaf(x[u], x[u], sq); }
    Vec4<float>::store(qs + c, x);
  }
  for (int c = tid * 4; c < kw; c += nt * 4) {
    float x[4], bb[4] = {0.f, 0.f, 0.f, 0.f};
    Vec4<T>::load(k + c, x);
    if (kb) Vec4<bf16>::load(kb + c, bb);
#pragma unroll
    for (int u = 0; u < 4; ++u) { x[u] += bb[u]; sk = fmaf(x[u], x[u], sk); }
    Vec4<float>::store(ks + c, x);
  }
  for (int c = tid * 4; c < vw; c += nt * 4) {
    float x[4], bb[4] = {0.f, 0.f, 0.f, 0.f};
    Vec4<T>::load(v + c, x);
    if (vb) Vec4<bf16>::load(vb + c, bb);
#pragma unroll
    for (int u = 0; u < 4; ++u) x[u] += bb[u];
    Vec4<T>::store(crow + kw + c, x);
  }
  head_scales(p, qs, ks, sq, sk, red, hr, pos);                 // ends with a barrier: the staged rows and the table are complete
  for (int part = 0; part < 2; ++part) {
    const int width = part == 0 ? qw : kw;
    const float* src = part == 0 ? qs : ks;
    const bf16* nw = (const bf16*)(part == 0 ? p.q_norm_w : p.k_norm_w);
    const float* hrs = part == 0 ? hr : hr + p.H;
    T* dst = part == 0 ? q : crow;
    for (int c = tid * 4; c < width; c += nt * 4) {
      const int e = c % p.dk;                                    // the four entries lie in one head and on one side of every border
      const int wo0 = p.norm_per_head ? e - c : 0;               // weight index = column + wo0 (a per-head weight has dk entries)
      const float rs = hrs[c / p.dk];
      float x[4], w[4] = {1.f, 1.f, 1.f, 1.f};
      Vec4<float>::load(src + c, x);
      if (nw) Vec4<bf16>::load(nw + c + wo0, w);
#pragma unroll
      for (int u = 0; u < 4; ++u) x[u] *= rs * w[u];
      if (e < p.rot_dims) {
        const int other = e < half ? c + half : c - half, a = e < half ? e : e - half;
        float y[4], wo[4] = {1.f, 1.f, 1.f, 1.f};
        Vec4<float>::load(src + other, y);
        if (nw) Vec4<bf16>::load(nw + other + wo0, wo);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float o = y[u] * rs * wo[u];
          // first half: u cos - v sin with v the partner; second half: v cos + u sin with u the partner
          x[u] = e < half ? x[u] * cs[a + u] - o * cs[half + a + u] : x[u] * cs[a + u] + o * cs[half + a + u];
        }
      }
      Vec4<T>::store(dst + c, x);
    }
  }
}

// grid (block slot, sequence): slot s is block pos / pool + s, done here iff its last row lies in [pos, pos + L)
template <typename T>
__global__ void __launch_bounds__(128) pool_rows_kernel(const T* __restrict__ cache, int64_t cache_row, int64_t cache_batch_stride, T* __restrict__ pooled,
                                                        int64_t pooled_row, int64_t pooled_batch_stride, int64_t L, int width, int64_t pool,
                                                        int64_t pos0, const int64_t* pos_dev) {
  const int64_t pos = pos_dev ? *pos_dev : pos0;
  const int64_t blk = pos / pool + blockIdx.x;
  const int64_t last = blk * pool + pool - 1;
  if (last < pos || last >= pos + L) return;
  const int b = blockIdx.y;
  const T* src = cache + (int64_t)b * cache_batch_stride + blk * pool * cache_row;
  T* dst = pooled + (int64_t)b * pooled_batch_stride + blk * pooled_row;
  const float inv = 1.0f / (float)pool;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = 0.f;
    for (int64_t r = 0; r < pool; ++r) s += ldf(src + r * cache_row + c);
    stf(dst + c, s * inv);
  }
}

}  // namespace

extern "C" int evo_qk_prep(const evo_qk_prep_params* p, void* stream) {
  EVO_REQUIRE(p->q && p->k && p->v && p->cache, "evo_qk_prep: null argument");
  EVO_REQUIRE(p->B >= 0 && p->L >= 0 && p->H > 0 && p->G > 0 && p->dk > 0 && p->dv > 0, "evo_qk_prep: bad shape");
  EVO_REQUIRE(p->rot_dims >= 0 && p->rot_dims <= p->dk && p->rot_dims % 2 == 0 && (p->rot_dims == 0 || p->freq), "evo_qk_prep: bad rotation (%d of %d)", p->rot_dims, p->dk);
  EVO_REQUIRE(p->cache_row >= (int64_t)p->G * (p->dk + p->dv), "evo_qk_prep: cache row too narrow");
  if (p->B == 0 || p->L == 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)(p->H + p->G) * p->dk + p->rot_dims + 4 + 33 + p->H + p->G);
  EVO_REQUIRE(smem <= 200 * 1024, "evo_qk_prep: projections too wide for one CTA's shared memory");
  const bool al = p->dtype ? aligned4<float>(p->q) && aligned4<float>(p->k) && aligned4<float>(p->v) && aligned4<float>(p->cache)
                           : aligned4<bf16>(p->q) && aligned4<bf16>(p->k) && aligned4<bf16>(p->v) && aligned4<bf16>(p->cache);
  const bool vec = al && p->dk % 4 == 0 && p->dv % 4 == 0 && p->rot_dims % 8 == 0 && p->ld % 4 == 0 && p->cache_row % 4 == 0 && p->cache_batch_stride % 4 == 0 &&
                   aligned4<bf16>(p->q_bias) && aligned4<bf16>(p->k_bias) && aligned4<bf16>(p->v_bias) && aligned4<bf16>(p->q_norm_w) && aligned4<bf16>(p->k_norm_w);
  auto kern = p->dtype ? (vec ? qk_prep4_kernel<float> : qk_prep_kernel<float>) : (vec ? qk_prep4_kernel<bf16> : qk_prep_kernel<bf16>);
  if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)((int64_t)p->B * p->L), 256, smem, (cudaStream_t)stream>>>(*p);
  return check_launch("evo_qk_prep");
}

extern "C" int evo_pool_rows(const void* cache, int64_t cache_row, int64_t cache_batch_stride, void* pooled, int64_t pooled_row, int64_t pooled_batch_stride,
                             int B, int64_t L, int width, int64_t pool, int64_t pos0, const int64_t* pos_dev, int dtype, void* stream) {
  EVO_REQUIRE(cache && pooled && pool > 0 && width > 0 && B >= 0 && L >= 0, "evo_pool_rows: bad arguments");
  if (B == 0 || L == 0) return 0;
  const dim3 grid((unsigned)(L / pool + 2), B);       // blocks that can end inside any L consecutive positions
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype) pool_rows_kernel<float><<<grid, 128, 0, st>>>((const float*)cache, cache_row, cache_batch_stride, (float*)pooled, pooled_row, pooled_batch_stride, L, width, pool, pos0, pos_dev);
  else pool_rows_kernel<bf16><<<grid, 128, 0, st>>>((const bf16*)cache, cache_row, cache_batch_stride, (bf16*)pooled, pooled_row, pooled_batch_stride, L, width, pool, pos0, pos_dev);
  return check_launch("evo_pool_rows");
}
