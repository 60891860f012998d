// Expert router of a mixture-of-experts feed-forward: fp32 logits W.h, scores by a softmax over all experts or a sigmoid per expert, the
// `top` experts with the largest (score + correction) are chosen -- optionally only inside the best groups of neighbouring experts -- and the
// output weights are the chosen experts' uncorrected scores times a constant, optionally divided by their sum first.  Further router rows
// give sigmoid gates that ride along (the gate of an always-on expert).  The dense weight row (0 for experts that were not chosen) is what the grouped activation kernel multiplies into
// the expert columns, so that the experts' weighted sum is the K-reduction of one down-projection GEMM.
//
// Prompts run only the chosen experts: (token, choice) pairs are counted per expert and given slots in expert order (evo_moe_count,
// evo_moe_scatter), the rows are gathered (evo_gather_rows), each expert runs its GEMMs on its slice, and evo_moe_combine adds the weighted
// rows back per token.
//
// A CTA of 8 warps owns TOK tokens (8 in a prompt, 1 in a decoding step, so that few tokens still spread over the GPU): warp w
// computes the logits of experts w, w + 8, ... for all of the CTA's tokens -- every router row it loads serves TOK tokens, the
// lanes split the row -- then warp t finishes token t (softmax, choice, weights).
#include "common.cuh"
#include "../../include/evo_b200.h"
#include <math.h>

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int RW = 8;         // warps per CTA

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf_lo(u.x), bf_hi(u.x), bf_lo(u.y), bf_hi(u.y));
}

// everything about one routing call that is not a pointer to rows
struct RouteArgs {
  const bf16* rw; const bf16* corr; float* weights; int64_t ldw; int32_t* chosen;
  int64_t rows; int D, E, top, n_extra, score_fn, groups, keep, normalize; float norm_eps, scale;
};

template <typename T, bool VEC, int TOK>
__global__ void __launch_bounds__(RW * 32) moe_route_kernel(const T* __restrict__ h, int64_t ldh, RouteArgs a) {
  extern __shared__ float sm[];             // [TOK][2 E + n_extra + 2 groups]: scores (then the extra rows' logits), selection scores, group ranks, group flags
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = a.E, D = a.D, NL = E + a.n_extra, per_tok = 2 * E + a.n_extra + 2 * a.groups;
  const int64_t row0 = (int64_t)blockIdx.x * TOK;
  const int nt = (int)min((int64_t)TOK, a.rows - row0);
  for (int e = w; e < NL; e += RW) {
    const bf16* wr = a.rw + (int64_t)e * D;
    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
    if (VEC) {                               // D % 4 == 0, rows aligned for 4-element accesses
#pragma unroll 2
      for (int k = lane * 4; k < D; k += 128) {
        const float4 w4 = ld4(wr + k);
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          const float4 h4 = ld4(h + (row0 + (t < nt ? t : 0)) * ldh + k);
          acc[t] = fmaf(h4.x, w4.x, fmaf(h4.y, w4.y, fmaf(h4.z, w4.z, fmaf(h4.w, w4.w, acc[t]))));
        }
      }
    } else {
      for (int k = lane; k < D; k += 32) {
        const float wv = __bfloat162float(wr[k]);
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc[t] = fmaf(ldf(h + (row0 + (t < nt ? t : 0)) * ldh + k), wv, acc[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      float d = acc[t];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) sm[t * per_tok + (e < E ? e : E + (e - E))] = d;       // experts at [0, E), extra rows at [E, E + n_extra)
    }
  }
  __syncthreads();
  for (int t = w; t < nt; t += RW) {
    float* s = sm + (size_t)t * per_tok;
    float* x = s + E;                        // extra rows' logits
    float* c = x + a.n_extra;                // selection scores
    float* rank = c + E;                     // [groups]
    float* kept = rank + a.groups;           // [groups]
    const int64_t row = row0 + t;
    if (a.score_fn == 0) {
      float mx = -INFINITY;
      for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
      for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - mx); s[e] = v; sum += v; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float inv = 1.f / sum;
      for (int e = lane; e < E; e += 32) s[e] *= inv;
    } else {
      for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-s[e]));
    }
    float* wrow = a.weights + row * a.ldw;
    for (int e = lane; e < E; e += 32) {
      c[e] = s[e] + (a.corr ? __bfloat162float(a.corr[e]) : 0.f);
      wrow[e] = 0.f;
    }
    for (int e = lane; e < a.n_extra; e += 32) wrow[E + e] = 1.f / (1.f + expf(-x[e]));
    __syncwarp();
    if (a.groups > 1) {
      // a run's rank: the sum of its two largest selection scores; the `keep` best runs stay, the others' experts cannot be chosen
      const int per = E / a.groups;
      for (int g = lane; g < a.groups; g += 32) {
        float b0 = -INFINITY, b1 = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float v = c[e];
          if (v > b0) { b1 = b0; b0 = v; } else if (v > b1) b1 = v;
        }
        rank[g] = per > 1 ? b0 + b1 : b0;
        kept[g] = 0.f;
      }
      __syncwarp();
      for (int k = 0; k < a.keep; ++k) {
        float best = -INFINITY; int bi = a.groups;
        for (int g = lane; g < a.groups; g += 32) if (kept[g] == 0.f && (rank[g] > best || bi == a.groups)) { best = rank[g]; bi = g; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (oi < a.groups && (bi == a.groups || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        if (lane == 0 && bi < a.groups) kept[bi] = 1.f;
        __syncwarp();
      }
      for (int e = lane; e < E; e += 32) if (kept[e / per] == 0.f) c[e] = -INFINITY;
      __syncwarp();
    }
    float picked = 0.f;                      // lane 0: sum of the chosen experts' scores
    for (int k = 0; k < a.top; ++k) {
      float best = -INFINITY; int bi = E;
      for (int e = lane; e < E; e += 32) if (c[e] > best) { best = c[e]; bi = e; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (lane == 0 && bi < E) {
        wrow[bi] = s[bi];
        picked += s[bi];
        c[bi] = -INFINITY;
        if (a.chosen) a.chosen[row * a.top + k] = bi;
      }
      __syncwarp();
    }
    picked = __shfl_sync(0xffffffffu, picked, 0);
    const float mul = a.normalize ? a.scale / (picked + a.norm_eps) : a.scale;
    for (int e = lane; e < E; e += 32) wrow[e] *= mul;
  }
}

template <typename T, bool VEC>
void launch(const T* h, int64_t ldh, const RouteArgs& a, cudaStream_t st) {
  const size_t per_tok = sizeof(float) * (2 * (size_t)a.E + a.n_extra + 2 * (size_t)a.groups);
  if (a.rows >= 1024) {
    constexpr int TOK = 8;
    moe_route_kernel<T, VEC, TOK><<<(unsigned)((a.rows + TOK - 1) / TOK), RW * 32, TOK * per_tok, st>>>(h, ldh, a);
  } else {
    moe_route_kernel<T, VEC, 1><<<(unsigned)a.rows, RW * 32, per_tok, st>>>(h, ldh, a);
  }
}

// ---- sparse execution of the chosen experts (prompts): rows sorted by expert, one GEMM pair per expert, weighted gather back
// counts[e] += 1 per (token, choice)
__global__ void moe_count_kernel(const int32_t* __restrict__ chosen, int64_t n, int E, int32_t* __restrict__ counts) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { const int e = chosen[i]; if (e >= 0 && e < E) atomicAdd(counts + e, 1); }
}
// slot of every (token, choice) in the expert-sorted order: offsets[e] + a running cursor (the order inside an expert is free: rows are
// independent); perm[slot] = token, slot_of[token, choice] = slot
__global__ void moe_scatter_kernel(const int32_t* __restrict__ chosen, int64_t n, int top, int E, const int32_t* __restrict__ offsets, int32_t* __restrict__ cursor,
                                   int32_t* __restrict__ perm, int32_t* __restrict__ slot_of) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = chosen[i];
  if (e < 0 || e >= E) { slot_of[i] = -1; return; }
  const int slot = offsets[e] + atomicAdd(cursor + e, 1);
  perm[slot] = (int32_t)(i / top);
  slot_of[i] = slot;
}
// dst[r, :] = src[perm[r], :]   (16-byte chunks; width_bytes % 16 == 0)
__global__ void gather_rows_kernel(const uint4* __restrict__ src, int64_t ld_src16, uint4* __restrict__ dst, int64_t ld_dst16, const int32_t* __restrict__ perm, int width16) {
  const int64_t r = blockIdx.x;
  const uint4* s = src + (int64_t)perm[r] * ld_src16;
  uint4* d = dst + r * ld_dst16;
  for (int c = threadIdx.x; c < width16; c += blockDim.x) d[c] = s[c];
}
// out[t, :] = base[t, :] + sum_k weights[t, chosen[t, k]] * ys[slot_of[t, k], :]   (fp32 sums; columns [D, ldo) zero)
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T* __restrict__ ys, int64_t ldy, const T* __restrict__ base, int64_t ldb, const float* __restrict__ weights,
                                                          int64_t ldw, int base_w, const int32_t* __restrict__ chosen, const int32_t* __restrict__ slot_of, T* __restrict__ out, int64_t ldo,
                                                          int D, int E, int top) {
  const int64_t t = blockIdx.x;
  const float bw = base_w ? weights[t * ldw + E] : 1.f;
  for (int c = threadIdx.x * 2; c < ldo; c += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    if (c < D) {
      if (base) { a0 = bw * ldf(base + t * ldb + c); a1 = c + 1 < D ? bw * ldf(base + t * ldb + c + 1) : 0.f; }
      for (int k = 0; k < top; ++k) {
        const int slot = slot_of[t * top + k];
        if (slot < 0) continue;
        const float w = weights[t * ldw + chosen[t * top + k]];
        a0 = fmaf(w, ldf(ys + (int64_t)slot * ldy + c), a0);
        if (c + 1 < D) a1 = fmaf(w, ldf(ys + (int64_t)slot * ldy + c + 1), a1);
      }
    }
    stf(out + t * ldo + c, a0);
    stf(out + t * ldo + c + 1, a1);
  }
}

}  // namespace

extern "C" int evo_moe_route_ex(const evo_moe_route_params* p, void* stream) {
  EVO_REQUIRE(p->h && p->router_w && p->weights && p->D > 0 && p->E > 0 && p->top > 0 && p->top <= p->E && p->ldh >= p->D && p->n_extra >= 0 &&
              p->ldw >= p->E + p->n_extra, "evo_moe_route: bad arguments");
  EVO_REQUIRE(p->E <= 512 && p->n_extra <= 64, "evo_moe_route: at most 512 experts and 64 further rows");
  EVO_REQUIRE(p->score_fn == 0 || p->score_fn == 1, "evo_moe_route: score function %d", p->score_fn);
  const int groups = p->groups > 1 ? p->groups : 0;
  EVO_REQUIRE(groups == 0 || (p->E % groups == 0 && p->keep > 0 && p->keep <= groups && (int64_t)p->keep * (p->E / groups) >= p->top),
              "evo_moe_route: %d experts in %d groups of which %d stay cannot give %d choices", p->E, groups, p->keep, p->top);
  if (p->rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = p->D % 4 == 0 && p->ldh % 4 == 0 && ((uintptr_t)p->h & (p->dtype ? 15 : 7)) == 0 && ((uintptr_t)p->router_w & 7) == 0;
  RouteArgs a = {(const bf16*)p->router_w, (const bf16*)p->correction, p->weights, p->ldw, p->chosen, p->rows, p->D, p->E, p->top, p->n_extra,
                 p->score_fn, groups, p->keep, p->normalize, p->norm_eps, p->scale};
  if (p->dtype) {
    if (vec) launch<float, true>((const float*)p->h, p->ldh, a, st); else launch<float, false>((const float*)p->h, p->ldh, a, st);
  } else {
    if (vec) launch<bf16, true>((const bf16*)p->h, p->ldh, a, st); else launch<bf16, false>((const bf16*)p->h, p->ldh, a, st);
  }
  return check_launch("evo_moe_route");
}

extern "C" int evo_moe_route(const void* h, int64_t ldh, const void* router_w, const void* correction, float* weights, int32_t* chosen,
                             int64_t rows, int D, int E, int top, float scale, int dtype, void* stream) {
  evo_moe_route_params p = {};
  p.h = h; p.ldh = ldh; p.router_w = router_w; p.correction = correction; p.weights = weights; p.ldw = E; p.chosen = chosen;
  p.rows = rows; p.D = D; p.E = E; p.top = top; p.scale = scale; p.dtype = dtype;
  return evo_moe_route_ex(&p, stream);
}

extern "C" int evo_moe_count(const int32_t* chosen, int64_t n, int E, int32_t* counts, void* stream) {
  EVO_REQUIRE(chosen && counts && E > 0, "evo_moe_count: bad arguments");
  if (n == 0) return 0;
  moe_count_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(chosen, n, E, counts);
  return check_launch("evo_moe_count");
}

extern "C" int evo_moe_scatter(const int32_t* chosen, int64_t n, int top, int E, const int32_t* offsets, int32_t* cursor, int32_t* perm, int32_t* slot_of, void* stream) {
  EVO_REQUIRE(chosen && offsets && cursor && perm && slot_of && top > 0 && E > 0, "evo_moe_scatter: bad arguments");
  if (n == 0) return 0;
  moe_scatter_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(chosen, n, top, E, offsets, cursor, perm, slot_of);
  return check_launch("evo_moe_scatter");
}

extern "C" int evo_gather_rows(const void* src, int64_t ld_src_bytes, void* dst, int64_t ld_dst_bytes, const int32_t* perm, int64_t rows, int64_t width_bytes, void* stream) {
  EVO_REQUIRE(src && dst && perm && width_bytes > 0, "evo_gather_rows: bad arguments");
  EVO_REQUIRE(width_bytes % 16 == 0 && ld_src_bytes % 16 == 0 && ld_dst_bytes % 16 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0,
              "evo_gather_rows: rows must be 16-byte aligned multiples of 16 bytes");
  if (rows == 0) return 0;
  gather_rows_kernel<<<(unsigned)rows, 128, 0, (cudaStream_t)stream>>>((const uint4*)src, ld_src_bytes / 16, (uint4*)dst, ld_dst_bytes / 16, perm, (int)(width_bytes / 16));
  return check_launch("evo_gather_rows");
}

extern "C" int evo_moe_combine(const void* ys, int64_t ldy, const void* base, int64_t ldb, const float* weights, int64_t ldw, int base_w, const int32_t* chosen, const int32_t* slot_of,
                               void* out, int64_t ldo, int64_t rows, int D, int E, int top, int dtype, void* stream) {
  EVO_REQUIRE(ys && weights && chosen && slot_of && out && D > 0 && ldy >= D && ldo >= D && ldo % 2 == 0 && (base == nullptr || ldb >= D), "evo_moe_combine: bad arguments");
  if (rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype) moe_combine_kernel<float><<<(unsigned)rows, 256, 0, st>>>((const float*)ys, ldy, (const float*)base, ldb, weights, ldw, base_w, chosen, slot_of, (float*)out, ldo, D, E, top);
  else moe_combine_kernel<bf16><<<(unsigned)rows, 256, 0, st>>>((const bf16*)ys, ldy, (const bf16*)base, ldb, weights, ldw, base_w, chosen, slot_of, (bf16*)out, ldo, D, E, top);
  return check_launch("evo_moe_combine");
}
