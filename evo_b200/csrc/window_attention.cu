// Softmax attention over a linear key/value cache with (a) a sliding window that also keeps the first tokens of the
// sequence, (b) one or two score maps per head over the same values (differential attention: o = a1 - lambda * a2),
// (c) an optional per-head RMS norm without weight, (d) an optional sigmoid output gate, (e) optionally soft-capped scores, a learned
// sink in the softmax denominator, a per-head bias that grows with the logarithm of the distance and, before the window, one pooled
// key/value per block of tokens -- one fused kernel; the
// scores, the softmax weights, the combination of the maps and the head norm are fp32 whatever the activation type.
//
// Work per query is bounded by window + keep_first keys, so the kernel is a CUDA-core streaming-softmax kernel: one warp
// per query, 8 consecutive queries per CTA share every 32-key tile of K and V through shared memory (their windows overlap
// almost completely); lane j scores key j of the tile against both maps, the probabilities are broadcast by shuffle and each
// lane accumulates dv/32 value channels.  A CTA only walks the tiles of [0, keep_first) and of the union of its windows.
// With few queries (the single-token step) the warps of a CTA split the key tiles of ONE query instead and merge their
// partial softmax states through shared memory.
#include "common.cuh"
#include "../../include/evo_b200.h"
#include <math.h>
#include <stdlib.h>

using namespace evo;

namespace evo {
int window_attn_mma(const evo_window_attn_params* p, cudaStream_t st);      // window_attention_mma.cu; 1 = shape not covered
}

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
// 16 bytes of a row as floats (EV = 16 / sizeof(T) elements), and 4 consecutive elements (8 bytes of bf16, 16 of fp32)
template <typename T> struct Row16;
template <> struct Row16<float> {
  static constexpr int EV = 4;
  static __device__ __forceinline__ void load(const float* p, float* o) { const float4 u = *reinterpret_cast<const float4*>(p); o[0] = u.x; o[1] = u.y; o[2] = u.z; o[3] = u.w; }
  static __device__ __forceinline__ void load4(const float* p, float* o) { load(p, o); }
};
template <> struct Row16<bf16> {
  static constexpr int EV = 8;
  static __device__ __forceinline__ void unpack(uint32_t u, float& a, float& b) { a = __uint_as_float(u << 16); b = __uint_as_float(u & 0xffff0000u); }
  static __device__ __forceinline__ void load(const bf16* p, float* o) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    unpack(u.x, o[0], o[1]); unpack(u.y, o[2], o[3]); unpack(u.z, o[4], o[5]); unpack(u.w, o[6], o[7]);
  }
  static __device__ __forceinline__ void load4(const bf16* p, float* o) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    unpack(u.x, o[0], o[1]); unpack(u.y, o[2], o[3]);
  }
};

constexpr int QT = 8;        // warps per CTA
constexpr int KT = 32;       // keys per tile (one per lane)
constexpr int QS_MAX = 16;   // most warps of the few-query kernel

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// soft cap of a scaled score: cap * tanh(s / cap), off when cap <= 0
__device__ __forceinline__ float capped(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }
// what the distance between query and key takes off the score: r1 ln(1 + r2 (i - j)); r1 = 0 when the head has no such bias
__device__ __forceinline__ float distance_bias(float r1, float r2, int64_t dist) { return r1 != 0.f ? r1 * logf(1.f + r2 * (float)dist) : 0.f; }
__device__ __forceinline__ void distance_numbers(const evo_window_attn_params& p, int h, float& r1, float& r2) {
  r1 = p.dist_r1 ? __bfloat162float(((const bf16*)p.dist_r1)[h]) : 0.f;
  r2 = p.dist_r1 ? __bfloat162float(((const bf16*)p.dist_r2)[h]) : 0.f;
}
// pooled blocks that position i sees: those that end at or before i - window
__device__ __forceinline__ int64_t blocks_seen(int64_t i, int64_t window, int64_t pool) {
  const int64_t n = i - window + 1;
  return (pool > 0 && window > 0 && n > 0) ? n / pool : 0;
}

template <int NM, int MAXCV>      // MAXCV: value channels per lane (dv <= 32 * MAXCV)
struct Softmax {
  float m[NM], l[NM], acc[NM][MAXCV];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int a = 0; a < NM; ++a) {
      m[a] = -INFINITY; l[a] = 0.f;
#pragma unroll
      for (int c = 0; c < MAXCV; ++c) acc[a][c] = 0.f;
    }
  }
};

// scores of this lane's key for all maps -> running max / sum update; returns the lane's probabilities in pm
template <int NM, int MAXCV>
__device__ __forceinline__ bool tile_scores(Softmax<NM, MAXCV>& sm, const float* qrow, const float* krow, int dk, float scale, float cap, float bias, bool vis, float* pm) {
  float s[NM];
#pragma unroll
  for (int a = 0; a < NM; ++a) {
    float d = 0.f;
    for (int e = 0; e < dk; ++e) d = fmaf(qrow[a * dk + e], krow[a * dk + e], d);
    s[a] = vis ? capped(d * scale, cap) - bias : -INFINITY;
  }
  if (!__any_sync(0xffffffffu, vis)) return false;
#pragma unroll
  for (int a = 0; a < NM; ++a) {
    const float mn = fmaxf(sm.m[a], warp_max(s[a]));
    const float corr = expf(sm.m[a] - mn);
    pm[a] = vis ? expf(s[a] - mn) : 0.f;
    sm.l[a] = sm.l[a] * corr + warp_sum(pm[a]);
    sm.m[a] = mn;
#pragma unroll
    for (int c = 0; c < MAXCV; ++c) sm.acc[a][c] *= corr;
  }
  return true;
}

// combination of the maps, head norm, gate, store (one warp = one query row)
// BLOCKED: accumulator c of a lane is channel lane * MAXCV + c (the vector path of the few-query kernel), else lane + 32 * c
template <typename T, int NM, int MAXCV, bool BLOCKED = false>
__device__ __forceinline__ void finish_row(const evo_window_attn_params& p, const Softmax<NM, MAXCV>& sm, int64_t row, int h, int lane) {
  const int dv = p.dv;
  float o[MAXCV];
  float ss = 0.f;
  // a sink adds exp(sink_h) to the denominator: with mx = max(m, sink), acc / l becomes acc e^(m-mx) / (l e^(m-mx) + e^(sink-mx))
  float num[NM], den[NM];
#pragma unroll
  for (int a = 0; a < NM; ++a) {
    num[a] = 1.f; den[a] = sm.l[a];
    if (p.sink) {
      const float sk = __bfloat162float(((const bf16*)p.sink)[h]);
      const float mx = fmaxf(sm.m[a], sk);
      num[a] = expf(sm.m[a] - mx);
      den[a] = fmaf(sm.l[a], num[a], expf(sk - mx));
    }
  }
#pragma unroll
  for (int c = 0; c < MAXCV; ++c) {
    float v = sm.acc[0][c] * num[0] / den[0];
    if (NM == 2) v -= p.lambda * (sm.acc[NM - 1][c] * num[NM - 1] / den[NM - 1]);
    o[c] = ((BLOCKED ? lane * MAXCV + c : lane + 32 * c) < dv) ? v : 0.f;
    ss = fmaf(o[c], o[c], ss);
  }
  float mul = 1.f;
  if (p.head_norm) mul = p.out_scale / sqrtf(warp_sum(ss) / (float)dv + p.norm_eps);
  T* orow = (T*)p.out + row * p.ldo;
  const T* grow = (p.gate && !p.gate_per_head) ? (const T*)p.gate + row * p.gate_tok_stride + h * dv : nullptr;
  if (p.gate && p.gate_per_head) mul *= 1.f / (1.f + expf(-ldf((const T*)p.gate + row * p.gate_tok_stride + h)));
#pragma unroll
  for (int c = 0; c < MAXCV; ++c) {
    const int ch = BLOCKED ? lane * MAXCV + c : lane + 32 * c;
    if (ch < dv) {
      float v = o[c] * mul;
      if (grow) v *= 1.f / (1.f + expf(-ldf(grow + ch)));
      stf(orow + h * dv + ch, v);
    }
  }
  if (h == p.H - 1)
    for (int64_t c = (int64_t)p.H * dv + lane; c < p.ldo; c += 32) stf(orow + c, 0.f);
}

// ---- many queries: one warp per query, K/V tiles shared by the CTA's 8 consecutive queries
template <typename T, int NM, int MAXCV>
__global__ void __launch_bounds__(QT * 32) window_attn_kernel(evo_window_attn_params p) {
  extern __shared__ float smem[];
  const int dk = p.dk, dv = p.dv, kw = NM * dk, kst = kw + 1;
  float* Ks = smem;                       // [KT][kw + 1]
  float* Vs = Ks + KT * kst;              // [KT][dv]
  float* Qs = Vs + KT * dv;               // [QT][kw]
  const int b = blockIdx.z, h = blockIdx.y, g = h / (p.H / p.G);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t pos = p.pos_dev ? (int64_t)*p.pos_dev : p.q_pos0;
  const int64_t rel0 = (int64_t)blockIdx.x * QT;
  const int64_t rel = rel0 + w;
  const bool valid = rel < p.Lq;
  const int64_t i = pos + rel;
  const int64_t row = (int64_t)b * p.Lq + rel;
  if (valid) {
    const T* q = (const T*)p.q + row * p.q_tok_stride + (int64_t)h * kw;
    for (int e = lane; e < kw; e += 32) Qs[w * kw + e] = ldf(q + e);
  }
  const T* kb = (const T*)p.k + (int64_t)b * p.k_batch_stride + (int64_t)g * kw;
  const T* vb = (const T*)p.v + (int64_t)b * p.v_batch_stride + (int64_t)g * dv;
  const int64_t i_lo = pos + rel0, i_hi = pos + min(p.Lq - 1, rel0 + QT - 1);
  const bool windowed = p.window > 0;
  const int64_t win_lo = windowed ? max((int64_t)0, i_lo - p.window + 1) : 0;
  const int64_t keep_hi = windowed ? min(p.keep_first, win_lo) : 0;
  const int64_t pool_hi = blocks_seen(i_hi, p.window, p.pool);          // pooled rows any query of this CTA sees
  const int64_t my_blocks = blocks_seen(i, p.window, p.pool);
  const T* pkb = pool_hi ? (const T*)p.pool_k + (int64_t)b * p.pool_batch_stride + (int64_t)g * kw : nullptr;
  const T* pvb = pool_hi ? (const T*)p.pool_v + (int64_t)b * p.pool_batch_stride + (int64_t)g * dv : nullptr;

  float r1, r2;
  distance_numbers(p, h, r1, r2);
  Softmax<NM, MAXCV> sm;
  sm.init();
  for (int part = 0; part < 3; ++part) {                  // kept first tokens, pooled blocks, window
    const int64_t lo = part == 2 ? win_lo : 0, hi = part == 0 ? keep_hi : (part == 1 ? pool_hi : i_hi + 1);       // rows [lo, hi)
    const T* kbase = part == 1 ? pkb : kb;
    const T* vbase = part == 1 ? pvb : vb;
    const int64_t kstr = part == 1 ? p.pool_tok_stride : p.k_tok_stride, vstr = part == 1 ? p.pool_tok_stride : p.v_tok_stride;
    for (int64_t k0 = lo; k0 < hi; k0 += KT) {
      const int nk = (int)min((int64_t)KT, hi - k0);
      __syncthreads();
      for (int idx = threadIdx.x; idx < nk * kw; idx += QT * 32) {
        const int r = idx / kw, e = idx % kw;
        Ks[r * kst + e] = ldf(kbase + (k0 + r) * kstr + e);
      }
      for (int idx = threadIdx.x; idx < nk * dv; idx += QT * 32) {
        const int r = idx / dv, e = idx % dv;
        Vs[r * dv + e] = ldf(vbase + (k0 + r) * vstr + e);
      }
      __syncthreads();
      if (!valid) continue;
      const int64_t kj = k0 + lane;
      const bool vis = lane < nk && (part == 1 ? kj < my_blocks : (kj <= i && (!windowed || i - kj < p.window || kj < p.keep_first)));
      float pm[NM];
      const float bias = (vis && part != 1) ? distance_bias(r1, r2, i - kj) : 0.f;       // pooled blocks have no distance
      if (!tile_scores<NM, MAXCV>(sm, Qs + w * kw, Ks + (lane < nk ? lane : 0) * kst, dk, p.scale, p.softcap, bias, vis, pm)) continue;
      for (int r = 0; r < nk; ++r) {
        float pr[NM];
#pragma unroll
        for (int a = 0; a < NM; ++a) pr[a] = __shfl_sync(0xffffffffu, pm[a], r);
#pragma unroll
        for (int c = 0; c < MAXCV; ++c) {
          const int ch = lane + 32 * c;
          if (ch < dv) {
            const float vv = Vs[r * dv + ch];
#pragma unroll
            for (int a = 0; a < NM; ++a) sm.acc[a][c] = fmaf(pr[a], vv, sm.acc[a][c]);
          }
        }
      }
    }
  }
  if (valid) finish_row<T, NM, MAXCV>(p, sm, row, h, lane);
}

// ---- few queries: one CTA per (query, head); its warps take the key tiles round-robin, straight from global memory
// VEC (head sizes, strides and bases allow 16-byte key loads and 4-channel value loads): same sums in the same order, fewer and
// wider loads -- the step is bound by streaming the window's keys and values once
template <typename T, int NM, int MAXCV, bool VEC>
__global__ void __launch_bounds__(QS_MAX * 32) window_attn_split_kernel(evo_window_attn_params p) {
  extern __shared__ float smem[];
  const int dk = p.dk, dv = p.dv, kw = NM * dk;
  float* Qs = smem;                                   // [kw]
  float* Mg = Qs + kw;                                // [warps][NM][2 + dvp] partial (max, sum, acc)
  const int dvp = MAXCV * 32;
  const int b = blockIdx.z, h = blockIdx.y, g = h / (p.H / p.G);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int64_t pos = p.pos_dev ? (int64_t)*p.pos_dev : p.q_pos0;
  const int64_t rel = blockIdx.x, i = pos + rel, row = (int64_t)b * p.Lq + rel;
  const T* q = (const T*)p.q + row * p.q_tok_stride + (int64_t)h * kw;
  for (int e = threadIdx.x; e < kw; e += blockDim.x) Qs[e] = ldf(q + e);
  __syncthreads();
  const T* kb = (const T*)p.k + (int64_t)b * p.k_batch_stride + (int64_t)g * kw;
  const T* vb = (const T*)p.v + (int64_t)b * p.v_batch_stride + (int64_t)g * dv;
  const bool windowed = p.window > 0;
  const int64_t win_lo = windowed ? max((int64_t)0, i - p.window + 1) : 0;
  const int64_t keep_hi = windowed ? min(p.keep_first, win_lo) : 0;
  const int64_t n_keep = (keep_hi + KT - 1) / KT, n_win = (i + 1 - win_lo + KT - 1) / KT;
  const int64_t pool_hi = blocks_seen(i, p.window, p.pool), n_pool = (pool_hi + KT - 1) / KT;
  const T* pkb = pool_hi ? (const T*)p.pool_k + (int64_t)b * p.pool_batch_stride + (int64_t)g * kw : nullptr;
  const T* pvb = pool_hi ? (const T*)p.pool_v + (int64_t)b * p.pool_batch_stride + (int64_t)g * dv : nullptr;

  float r1, r2;
  distance_numbers(p, h, r1, r2);
  Softmax<NM, MAXCV> sm;
  sm.init();
  for (int64_t t = w; t < n_keep + n_pool + n_win; t += nw) {
    const bool pooled = t >= n_keep && t < n_keep + n_pool;
    const int64_t k0 = t < n_keep ? t * KT : (pooled ? (t - n_keep) * KT : win_lo + (t - n_keep - n_pool) * KT);
    const int64_t hi = t < n_keep ? keep_hi : (pooled ? pool_hi : i + 1);
    const int nk = (int)min((int64_t)KT, hi - k0);
    const bool vis = lane < nk;                        // every key of these ranges is visible to the one query
    const int64_t kstr = pooled ? p.pool_tok_stride : p.k_tok_stride, vstr = pooled ? p.pool_tok_stride : p.v_tok_stride;
    const T* vsrc = pooled ? pvb : vb;
    const T* krow = (pooled ? pkb : kb) + (k0 + (vis ? lane : 0)) * kstr;
    float s[NM], pm[NM];
#pragma unroll
    for (int a = 0; a < NM; ++a) {
      float d = 0.f;
      if (VEC) {
        constexpr int EV = Row16<T>::EV;
#pragma unroll 4
        for (int e = 0; e < dk; e += EV) {
          float kv[EV];
          Row16<T>::load(krow + a * dk + e, kv);
#pragma unroll
          for (int u = 0; u < EV; ++u) d = fmaf(Qs[a * dk + e + u], kv[u], d);
        }
      } else {
        for (int e = 0; e < dk; ++e) d = fmaf(Qs[a * dk + e], ldf(krow + a * dk + e), d);
      }
      s[a] = vis ? capped(d * p.scale, p.softcap) - ((vis && !pooled) ? distance_bias(r1, r2, i - (k0 + lane)) : 0.f) : -INFINITY;
    }
#pragma unroll
    for (int a = 0; a < NM; ++a) {
      const float mn = fmaxf(sm.m[a], warp_max(s[a]));
      const float corr = expf(sm.m[a] - mn);
      pm[a] = vis ? expf(s[a] - mn) : 0.f;
      sm.l[a] = sm.l[a] * corr + warp_sum(pm[a]);
      sm.m[a] = mn;
#pragma unroll
      for (int c = 0; c < MAXCV; ++c) sm.acc[a][c] *= corr;
    }
    if (VEC) {
      const bool mine = lane * MAXCV < dv;             // dv % 4 == 0: a lane's groups of 4 channels are inside the head or outside
#pragma unroll 8
      for (int r = 0; r < nk; ++r) {
        float pr[NM];
#pragma unroll
        for (int a = 0; a < NM; ++a) pr[a] = __shfl_sync(0xffffffffu, pm[a], r);
        const T* vrow = vsrc + (k0 + r) * vstr + lane * MAXCV;
#pragma unroll
        for (int c = 0; c < MAXCV; c += 4) {
          if (mine && lane * MAXCV + c < dv) {
            float vv[4];
            Row16<T>::load4(vrow + c, vv);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
              for (int a = 0; a < NM; ++a) sm.acc[a][c + u] = fmaf(pr[a], vv[u], sm.acc[a][c + u]);
          }
        }
      }
      continue;
    }
    for (int r = 0; r < nk; ++r) {
      float pr[NM];
#pragma unroll
      for (int a = 0; a < NM; ++a) pr[a] = __shfl_sync(0xffffffffu, pm[a], r);
      const T* vrow = vsrc + (k0 + r) * vstr;
#pragma unroll
      for (int c = 0; c < MAXCV; ++c) {
        const int ch = lane + 32 * c;
        if (ch < dv) {
          const float vv = ldf(vrow + ch);
#pragma unroll
          for (int a = 0; a < NM; ++a) sm.acc[a][c] = fmaf(pr[a], vv, sm.acc[a][c]);
        }
      }
    }
  }
  // merge the warps' partial states in warp 0
#pragma unroll
  for (int a = 0; a < NM; ++a) {
    float* dst = Mg + ((w * NM + a) * (2 + dvp));
    if (lane == 0) { dst[0] = sm.m[a]; dst[1] = sm.l[a]; }
#pragma unroll
    for (int c = 0; c < MAXCV; ++c) dst[2 + lane + 32 * c] = sm.acc[a][c];
  }
  __syncthreads();
  if (w != 0) return;
  Softmax<NM, MAXCV> tot;
  tot.init();
#pragma unroll
  for (int a = 0; a < NM; ++a) {
    float mx = -INFINITY;
    for (int ww = 0; ww < nw; ++ww) mx = fmaxf(mx, Mg[(ww * NM + a) * (2 + dvp)]);
    tot.m[a] = mx;
    for (int ww = 0; ww < nw; ++ww) {
      const float* src = Mg + (ww * NM + a) * (2 + dvp);
      if (src[0] == -INFINITY) continue;              // this warp saw no tile
      const float sc = expf(src[0] - mx);
      tot.l[a] = fmaf(src[1], sc, tot.l[a]);
#pragma unroll
      for (int c = 0; c < MAXCV; ++c) tot.acc[a][c] = fmaf(src[2 + lane + 32 * c], sc, tot.acc[a][c]);
    }
  }
  finish_row<T, NM, MAXCV, VEC>(p, tot, row, h, lane);
}

template <typename T, int NM, int MAXCV>
int launch_cv(const evo_window_attn_params* p, cudaStream_t st) {
  const int kw = NM * p->dk;
  if (p->Lq <= 4) {
    // the warps of a CTA take the query's key tiles in turn; each tile is a chain of dependent loads (keys -> weights -> values), so
    // a long window gets more warps: shorter chains and more bytes in flight
    int64_t span = p->window > 0 ? (int64_t)p->window + p->keep_first : (p->pos_dev ? (int64_t)1 << 30 : p->q_pos0 + p->Lq);
    if (p->pool > 0) span += p->pos_dev ? (int64_t)1 << 20 : (p->q_pos0 + p->Lq) / p->pool;
    const int warps = span >= 24 * KT ? QS_MAX : QT;
    const size_t smem = sizeof(float) * ((size_t)kw + (size_t)warps * NM * (2 + MAXCV * 32));
    constexpr int EV = Row16<T>::EV;
    auto a16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
    const bool vec = p->dk % EV == 0 && p->dv % 4 == 0 && p->k_tok_stride % EV == 0 && p->k_batch_stride % EV == 0 && p->v_tok_stride % EV == 0 &&
                     p->v_batch_stride % EV == 0 && a16(p->k) && a16(p->v) &&
                     (p->pool <= 0 || (p->pool_tok_stride % EV == 0 && p->pool_batch_stride % EV == 0 && a16(p->pool_k) && a16(p->pool_v)));
    auto kern = vec ? window_attn_split_kernel<T, NM, MAXCV, true> : window_attn_split_kernel<T, NM, MAXCV, false>;
    if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<dim3((unsigned)p->Lq, p->H, p->B), warps * 32, smem, st>>>(*p);
  } else {
    const size_t smem = sizeof(float) * ((size_t)KT * (kw + 1) + (size_t)KT * p->dv + (size_t)QT * kw);
    EVO_REQUIRE(smem <= 227 * 1024, "evo_window_attn_fwd: head too wide for shared memory (%zu bytes)", smem);
    auto kern = window_attn_kernel<T, NM, MAXCV>;
    if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<dim3((unsigned)((p->Lq + QT - 1) / QT), p->H, p->B), QT * 32, smem, st>>>(*p);
  }
  return check_launch("evo_window_attn_fwd");
}

template <typename T, int NM>
int launch(const evo_window_attn_params* p, cudaStream_t st) {
  if (p->dv <= 128) return launch_cv<T, NM, 4>(p, st);
  if (p->dv <= 256) return launch_cv<T, NM, 8>(p, st);
  return launch_cv<T, NM, 16>(p, st);
}

}  // namespace

extern "C" int evo_window_attn_fwd(const evo_window_attn_params* p, void* stream) {
  EVO_REQUIRE(p->q && p->k && p->v && p->out, "evo_window_attn_fwd: null argument");
  EVO_REQUIRE(p->B >= 0 && p->Lq >= 0 && p->H > 0 && p->G > 0 && p->H % p->G == 0 && p->dk > 0 && p->dv > 0, "evo_window_attn_fwd: bad shape");
  EVO_REQUIRE(p->n_maps == 1 || p->n_maps == 2, "evo_window_attn_fwd: n_maps must be 1 or 2");
  EVO_REQUIRE(p->dv <= 512, "evo_window_attn_fwd: dv (%d) must be <= 512", p->dv);
  EVO_REQUIRE(p->ldo >= (int64_t)p->H * p->dv, "evo_window_attn_fwd: ldo too small");
  EVO_REQUIRE(p->pool <= 0 || (p->window > 0 && p->pool_k && p->pool_v), "evo_window_attn_fwd: pooled blocks need a window and the pooled rows");
  EVO_REQUIRE((p->dist_r1 == nullptr) == (p->dist_r2 == nullptr), "evo_window_attn_fwd: the distance bias needs both of its numbers");
  if (p->B == 0 || p->Lq == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  static const char* env_mma = getenv("EVO_B200_WINDOW_ATTN_MMA");      // "0": always the CUDA-core kernel (comparisons)
  if (!(env_mma && atoi(env_mma) == 0)) {
    const int rc = window_attn_mma(p, st);                              // bf16, two maps, >= 16 query rows, heads up to 128
    if (rc <= 0) return rc;
  }
  if (p->dtype) return p->n_maps == 2 ? launch<float, 2>(p, st) : launch<float, 1>(p, st);
  return p->n_maps == 2 ? launch<bf16, 2>(p, st) : launch<bf16, 1>(p, st);
}
