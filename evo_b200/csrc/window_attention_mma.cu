// Tensor-core form of the windowed attention with one or two score maps (see window_attention.cu for the mechanism) for bf16 activations.
// The fp32 rule of the design is kept: scores are exact bf16 x bf16 products accumulated in fp32 (mma.sync m16n8k16), the softmax
// runs in fp32 registers, and each probability enters P.V as a bf16 high part plus a bf16 low part (two MMAs, relative error
// 2^-17 per weight instead of 2^-9), accumulated in fp32.
//
// CTA = 4 warps x 16 queries, 64-key tiles of K (both maps) and V in shared memory as bf16, row-major with 16-byte row padding
// (conflict-free fragment reads; V fragments come transposed out of ldmatrix), filled with 16-byte copies when the head sizes and
// strides are multiples of 8 -- asynchronous ones into two buffers, the next tile on its way while the current one is in work, as
// long as two CTAs still fit an SM's shared memory.  A warp keeps both maps' output accumulators (16 x dv fp32 each) in registers and handles one map
// at a time (scores -> softmax -> P.V), so only one 16 x 64 tile of probabilities is live.
// Head sizes are padded to 16 in shared memory (zero columns); dk <= 128, dv <= 128 and dv % 8 == 0, otherwise the CUDA-core
// kernel runs.  The tile walk is the CUDA-core kernel's: [0, keep_first), the pooled blocks that the CTA's last query sees, and the
// union of the CTA's windows.  A soft cap is applied to the fp32 scores before the softmax (tanh from ex2 and a division), and a
// sink enters the denominators at the end; a distance bias is taken off the fp32 scores together with the mask.
#include "common.cuh"
#include "mma_sync.cuh"
#include "../../include/evo_b200.h"
#include <math.h>

using namespace evo;

namespace evo {
int window_attn_mma(const evo_window_attn_params* p, cudaStream_t st);      // returns 1 when the shape is not covered
}

namespace {

constexpr int WARPS = 4, QROWS = 16, KT = 64;

// 16 bytes global -> shared without passing through registers; !live: 16 zero bytes (nothing is read)
__device__ __forceinline__ void copy16_async(void* dst, const void* src, bool live) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(live ? 16 : 0) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// NV8 = padded dv / 8 (output tiles of 8 channels per warp row block)
template <int NV8, int NM>
__global__ void __launch_bounds__(WARPS * 32) window_attn_mma_kernel(evo_window_attn_params p, int dkp, int qst, int kst, int vst, int vec, int2 vstep, int nbuf) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [WARPS*16][qst]   both maps' queries
  bf16* Ks0 = Qs + WARPS * QROWS * qst;                          // [nbuf][KT][kst]   both maps' keys
  bf16* Vs0 = Ks0 + nbuf * KT * kst;                             // [nbuf][KT][vst]   values
  const int dk = p.dk, dv = p.dv;
  const int b = blockIdx.z, h = blockIdx.y, g = h / (p.H / p.G);
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, qr = lane >> 2, qc = (lane & 3) * 2;
  const int64_t pos = p.pos_dev ? (int64_t)*p.pos_dev : p.q_pos0;
  const int64_t rel0 = (int64_t)blockIdx.x * (WARPS * QROWS);
  // 16-byte copies of [row][both maps' dkp columns]: a row has c8n chunks, cpm per map; this thread's first (row, chunk) and its step
  // (vstep = 128 / c8n, 128 % c8n, from the host) replace a division per copy
  const int cpm = dkp / 8, c8n = NM * cpm, vr0 = tid / c8n, vc0 = tid % c8n;
  const bf16* qg = (const bf16*)p.q;
  // queries of the CTA: [row][map][dkp], zero padding for rows past Lq and columns past dk
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  if (vec) {                              // dk, dv, strides multiples of 8 and 16-byte aligned bases: 8 elements per copy
    for (int r = vr0, cc = vc0; r < WARPS * QROWS; ) {
      const int m = cc >= cpm, e = (cc - m * cpm) * 8;
      const int64_t rel = rel0 + r;
      uint4 v = zero4;
      if (rel < p.Lq && e < dk) v = *reinterpret_cast<const uint4*>(qg + ((int64_t)b * p.Lq + rel) * p.q_tok_stride + (int64_t)h * NM * dk + m * dk + e);
      *reinterpret_cast<uint4*>(Qs + r * qst + cc * 8) = v;
      r += vstep.x; cc += vstep.y;
      if (cc >= c8n) { cc -= c8n; ++r; }
    }
  } else {
    for (int idx = tid; idx < WARPS * QROWS * NM * dkp; idx += WARPS * 32) {
      const int r = idx / (NM * dkp), c = idx % (NM * dkp), m = c / dkp, e = c % dkp;
      const int64_t rel = rel0 + r;
      bf16 v = __float2bfloat16_rn(0.f);
      if (rel < p.Lq && e < dk) v = qg[((int64_t)b * p.Lq + rel) * p.q_tok_stride + (int64_t)h * NM * dk + m * dk + e];
      Qs[r * qst + c] = v;
    }
  }
  const bf16* kb = (const bf16*)p.k + (int64_t)b * p.k_batch_stride + (int64_t)g * NM * dk;
  const bf16* vb = (const bf16*)p.v + (int64_t)b * p.v_batch_stride + (int64_t)g * dv;
  const int64_t i_lo = pos + rel0, i_hi = pos + min(p.Lq - 1, rel0 + WARPS * QROWS - 1);
  const bool windowed = p.window > 0;
  const int64_t win_lo = windowed ? max((int64_t)0, i_lo - p.window + 1) : 0;
  const int64_t keep_hi = windowed ? min(p.keep_first, win_lo) : 0;
  // this warp's rows
  const int64_t i0 = pos + rel0 + w * QROWS + qr, i1 = i0 + 8;                // positions of the thread's two rows
  const int64_t wi_lo = pos + rel0 + w * QROWS, wi_hi = wi_lo + QROWS - 1;     // the warp's first / last position

  float O[NM][NV8][4];
  float mrun[NM][2], lrun[NM][2];
#pragma unroll
  for (int m = 0; m < NM; ++m) {
    mrun[m][0] = mrun[m][1] = -INFINITY; lrun[m][0] = lrun[m][1] = 0.f;
#pragma unroll
    for (int n = 0; n < NV8; ++n) O[m][n][0] = O[m][n][1] = O[m][n][2] = O[m][n][3] = 0.f;
  }
  const bf16* Qw = Qs + (w * QROWS) * qst;
  const float LOG2E = 1.4426950408889634f;
  const float scale2 = p.scale * LOG2E;
  // soft cap: cap * tanh(s / cap) with tanh(x) = 1 - 2 / (2^(2 x log2 e) + 1), in base-2 units like the plain scores
  const bool capped = p.softcap > 0.f;
  const float cap_in = capped ? p.scale / p.softcap * 2.f * LOG2E : 0.f, cap_out = p.softcap * LOG2E;
  // pooled blocks before the window: block b is seen from position i iff b < (i - window + 1) / pool
  const auto seen = [&](int64_t i) -> int64_t { const int64_t n = i - p.window + 1; return (p.pool > 0 && n > 0) ? n / p.pool : 0; };
  const int64_t pool_hi = windowed ? seen(i_hi) : 0;
  const int64_t seen0 = windowed ? seen(i0) : 0, seen1 = windowed ? seen(i1) : 0, wseen_lo = windowed ? seen(wi_lo) : 0, wseen_hi = windowed ? seen(wi_hi) : 0;
  const bf16* pkb = pool_hi ? (const bf16*)p.pool_k + (int64_t)b * p.pool_batch_stride + (int64_t)g * NM * dk : nullptr;
  const bf16* pvb = pool_hi ? (const bf16*)p.pool_v + (int64_t)b * p.pool_batch_stride + (int64_t)g * dv : nullptr;
  // distance bias r1 ln(1 + r2 d), in base-2 units: r1 log2(1 + r2 d)
  const bool biased = p.dist_r1 != nullptr;
  const float r1 = biased ? __bfloat162float(((const bf16*)p.dist_r1)[h]) : 0.f, r2 = biased ? __bfloat162float(((const bf16*)p.dist_r2)[h]) : 0.f;

  int cur = 0;                                          // buffer of the tile in work
  for (int part = 0; part < 3; ++part) {               // kept first tokens, pooled blocks, window
    const int64_t lo = part == 2 ? win_lo : 0, hi = part == 0 ? keep_hi : (part == 1 ? pool_hi : i_hi + 1);
    const bool pooled = part == 1;
    const bf16* kbase = pooled ? pkb : kb;
    const bf16* vbase = pooled ? pvb : vb;
    const int64_t kstr = pooled ? p.pool_tok_stride : p.k_tok_stride, vstr = pooled ? p.pool_tok_stride : p.v_tok_stride;
    // the tile that starts at key t0, as asynchronous 16-byte copies into buffer `bufi` (one group per thread)
    const auto fetch = [&](int64_t t0, int bufi) {
      const int n = (int)min((int64_t)KT, hi - t0);
      bf16* Kd = Ks0 + bufi * KT * kst;
      bf16* Vd = Vs0 + bufi * KT * vst;
      for (int r = vr0, cc = vc0; r < KT; ) {
        const int m = cc >= cpm, e = (cc - m * cpm) * 8;
        const bool live = r < n && e < dk;
        copy16_async(Kd + r * kst + cc * 8, live ? kbase + (t0 + r) * kstr + m * dk + e : kbase, live);
        r += vstep.x; cc += vstep.y;
        if (cc >= c8n) { cc -= c8n; ++r; }
      }
      for (int idx = tid; idx < KT * NV8; idx += WARPS * 32) {
        const int r = idx / NV8, c = (idx % NV8) * 8;
        const bool live = r < n && c < dv;
        copy16_async(Vd + r * vst + c, live ? vbase + (t0 + r) * vstr + c : vbase, live);
      }
      copies_commit();
    };
    bool ahead = false;                                // the tile of this iteration was fetched during the previous one
    for (int64_t k0 = lo; k0 < hi; k0 += KT) {
      const int nk = (int)min((int64_t)KT, hi - k0);
      bf16* Ks = Ks0 + cur * KT * kst;
      bf16* Vs = Vs0 + cur * KT * vst;
      __syncthreads();                                 // every warp has left the previous tile: the other buffer may be overwritten
      if (vec) {
        if (!ahead) fetch(k0, cur);
        if (nbuf == 2 && k0 + KT < hi) { fetch(k0 + KT, cur ^ 1); ahead = true; copies_wait<1>(); }
        else { ahead = false; copies_wait<0>(); }
        if (nbuf == 2) cur ^= 1;
      } else {
        for (int idx = tid; idx < KT * NM * dkp; idx += WARPS * 32) {
          const int r = idx / (NM * dkp), c = idx % (NM * dkp), m = c / dkp, e = c % dkp;
          bf16 v = __float2bfloat16_rn(0.f);
          if (r < nk && e < dk) v = kbase[(k0 + r) * kstr + m * dk + e];
          Ks[r * kst + c] = v;
        }
        for (int idx = tid; idx < KT * NV8 * 8; idx += WARPS * 32) {
          const int r = idx / (NV8 * 8), c = idx % (NV8 * 8);
          bf16 v = __float2bfloat16_rn(0.f);
          if (r < nk && c < dv) v = vbase[(k0 + r) * vstr + c];
          Vs[r * vst + c] = v;
        }
      }
      __syncthreads();
      // a tile none of the warp's rows can see
      const int64_t t_lo = k0, t_hi = k0 + nk - 1;
      bool full;
      if (pooled) {
        if (t_lo >= wseen_hi) continue;
        full = nk == KT && t_hi < wseen_lo;
      } else {
        if (t_lo > wi_hi) continue;
        if (windowed && wi_lo - t_hi >= p.window && t_lo >= p.keep_first) continue;
        full = nk == KT && t_hi <= wi_lo && (!windowed || wi_hi - t_lo < p.window || t_hi < p.keep_first);
      }

#pragma unroll
      for (int m = 0; m < NM; ++m) {
        // scores of map m: S (16 x 64) = Q_m (16 x dkp) . K_m^T
        float Pm[1][KT / 8][4];
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) Pm[0][n][0] = Pm[0][n][1] = Pm[0][n][2] = Pm[0][n][3] = 0.f;
        for (int ks = 0; ks < dkp / 16; ++ks) {
          uint32_t a[4];
          const bf16* qa = Qw + m * dkp + ks * 16 + qc;
          a[0] = *reinterpret_cast<const uint32_t*>(qa + qr * qst);
          a[1] = *reinterpret_cast<const uint32_t*>(qa + (qr + 8) * qst);
          a[2] = *reinterpret_cast<const uint32_t*>(qa + qr * qst + 8);
          a[3] = *reinterpret_cast<const uint32_t*>(qa + (qr + 8) * qst + 8);
#pragma unroll
          for (int n = 0; n < KT / 8; n += 2) {
            uint32_t kf[4];            // b0, b1 of key tile n, then of tile n + 1: rows = keys, 8 features per 16-byte row
            ldmatrix_x4(kf, Ks + ((n + (lane >> 4)) * 8 + (lane & 7)) * kst + m * dkp + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(Pm[0][n], a, kf[0], kf[1]);
            mma_bf16(Pm[0][n + 1], a, kf[2], kf[3]);
          }
        }
        // mask, running max / sum, probabilities
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (full) {                                    // every key of the tile is visible to every row of the warp: no mask
          const int d0 = (int)(i0 - k0) - qc;          // distance of the row's first key column in the tile (the lower row is 8 further)
#pragma unroll
          for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              float s = capped ? cap_out * (1.f - __fdividef(2.f, ex2(Pm[0][n][c] * cap_in) + 1.f)) : Pm[0][n][c] * scale2;
              if (biased && !pooled) s = fmaf(-r1, __log2f(fmaf(r2, (float)(((c < 2) ? d0 : d0 + 8) - (n * 8 + (c & 1))), 1.f)), s);
              Pm[0][n][c] = s;
              if (c < 2) mx0 = fmaxf(mx0, s); else mx1 = fmaxf(mx1, s);
            }
          }
        } else
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int64_t kj = k0 + n * 8 + qc + (c & 1);
            const int64_t i = (c < 2) ? i0 : i1;
            const bool vis = (n * 8 + qc + (c & 1)) < nk &&
                             (pooled ? kj < ((c < 2) ? seen0 : seen1) : (kj <= i && (!windowed || i - kj < p.window || kj < p.keep_first)));
            const float sc = capped ? cap_out * (1.f - __fdividef(2.f, ex2(Pm[0][n][c] * cap_in) + 1.f)) : Pm[0][n][c] * scale2;
            float s = vis ? sc : -INFINITY;                                // base-2 exponent: exp(x) = 2^(x log2 e)
            if (biased && vis && !pooled) s = fmaf(-r1, __log2f(fmaf(r2, (float)(i - kj), 1.f)), s);
            Pm[0][n][c] = s;
            if (c < 2) mx0 = fmaxf(mx0, s); else mx1 = fmaxf(mx1, s);
          }
        }
        mx0 = quad_max(mx0); mx1 = quad_max(mx1);
        const float mn0 = fmaxf(mrun[m][0], mx0), mn1 = fmaxf(mrun[m][1], mx1);
        // rows that have seen no key yet keep max = -inf: use 0 as the reference so that exp() gives 0, not NaN
        const float r0 = mn0 == -INFINITY ? 0.f : mn0, r1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = ex2(mrun[m][0] - r0), c1 = ex2(mrun[m][1] - r1);
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) {
          Pm[0][n][0] = ex2(Pm[0][n][0] - r0); Pm[0][n][1] = ex2(Pm[0][n][1] - r0);
          Pm[0][n][2] = ex2(Pm[0][n][2] - r1); Pm[0][n][3] = ex2(Pm[0][n][3] - r1);
          s0 += Pm[0][n][0] + Pm[0][n][1]; s1 += Pm[0][n][2] + Pm[0][n][3];
        }
        lrun[m][0] = lrun[m][0] * c0 + quad_sum(s0); lrun[m][1] = lrun[m][1] * c1 + quad_sum(s1);
        const bool moved = !__all_sync(0xffffffffu, mn0 == mrun[m][0] && mn1 == mrun[m][1]);
        mrun[m][0] = mn0; mrun[m][1] = mn1;
        if (moved) {                                   // some row's maximum moved; otherwise c0 = c1 = 1 (or the row is still empty)
#pragma unroll
          for (int n = 0; n < NV8; ++n) { O[m][n][0] *= c0; O[m][n][1] *= c0; O[m][n][2] *= c1; O[m][n][3] *= c1; }
        }
        // O_m += P_m . V: high and low bf16 parts of P against the same V fragments (ldmatrix, transposed on the way)
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          uint32_t ah[4], al[4];
          split_pack(Pm[0][2 * kk][0], Pm[0][2 * kk][1], ah[0], al[0]);
          split_pack(Pm[0][2 * kk][2], Pm[0][2 * kk][3], ah[1], al[1]);
          split_pack(Pm[0][2 * kk + 1][0], Pm[0][2 * kk + 1][1], ah[2], al[2]);
          split_pack(Pm[0][2 * kk + 1][2], Pm[0][2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
          for (int n = 0; n < NV8; n += 2) {
            uint32_t bv[4];          // b0, b1 of channel tile n, then of tile n + 1
            ldmatrix_x4_trans(bv, Vs + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * vst + (n + (lane >> 4)) * 8);
            mma_bf16(O[m][n], ah, bv[0], bv[1]); mma_bf16(O[m][n], al, bv[0], bv[1]);
            mma_bf16(O[m][n + 1], ah, bv[2], bv[3]); mma_bf16(O[m][n + 1], al, bv[2], bv[3]);
          }
        }
      }
    }
  }
  // o = a1 / l1 - lambda * a2 / l2, head norm, gate, store
  const int64_t rel_a = rel0 + w * QROWS + qr, rel_b = rel_a + 8;
  float il[2][2] = {{1.f / lrun[0][0], 1.f / lrun[0][1]}, {1.f / lrun[NM - 1][0], 1.f / lrun[NM - 1][1]}};
  if (p.sink) {      // exp(sink_h) joins the denominator: with mx = max(m, sink), acc / l becomes acc 2^(m-mx) / (l 2^(m-mx) + 2^(sink-mx))
    const float sk = __bfloat162float(((const bf16*)p.sink)[h]) * LOG2E;
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int m = a == 0 ? 0 : NM - 1;
        const float mx = fmaxf(mrun[m][r], sk), num = ex2(mrun[m][r] - mx);
        il[a][r] = num / fmaf(lrun[m][r], num, ex2(sk - mx));
      }
  }
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int n = 0; n < NV8; ++n) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = c >> 1;
      float v = O[0][n][c] * il[0][r];
      if (NM == 2) v -= p.lambda * (O[NM - 1][n][c] * il[1][r]);
      const bool live = n * 8 + qc + (c & 1) < dv;
      O[0][n][c] = live ? v : 0.f;
      if (r == 0) ss0 = fmaf(O[0][n][c], O[0][n][c], ss0); else ss1 = fmaf(O[0][n][c], O[0][n][c], ss1);
    }
  }
  float mul0 = 1.f, mul1 = 1.f;
  if (p.head_norm) {
    mul0 = p.out_scale / sqrtf(quad_sum(ss0) / (float)dv + p.norm_eps);
    mul1 = p.out_scale / sqrtf(quad_sum(ss1) / (float)dv + p.norm_eps);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int64_t rel = r == 0 ? rel_a : rel_b;
    if (rel >= p.Lq) continue;
    const int64_t row = (int64_t)b * p.Lq + rel;
    bf16* orow = (bf16*)p.out + row * p.ldo + (int64_t)h * dv;
    const bf16* grow = (p.gate && !p.gate_per_head) ? (const bf16*)p.gate + row * p.gate_tok_stride + (int64_t)h * dv : nullptr;
    float mul = r == 0 ? mul0 : mul1;
    if (p.gate && p.gate_per_head) mul *= 1.f / (1.f + expf(-__bfloat162float(((const bf16*)p.gate)[row * p.gate_tok_stride + h])));
#pragma unroll
    for (int n = 0; n < NV8; ++n) {
      const int ch = n * 8 + qc;
      if (ch < dv) {                                   // dv is even: the pair (ch, ch + 1) is inside the head
        float v0 = O[0][n][2 * r] * mul, v1 = O[0][n][2 * r + 1] * mul;
        if (grow) {
          v0 *= 1.f / (1.f + expf(-__bfloat162float(grow[ch])));
          v1 *= 1.f / (1.f + expf(-__bfloat162float(grow[ch + 1])));
        }
        orow[ch] = __float2bfloat16_rn(v0);
        orow[ch + 1] = __float2bfloat16_rn(v1);
      }
    }
    if (h == p.H - 1)
      for (int64_t c = (int64_t)p.H * dv + (lane & 3); c < p.ldo; c += 4) ((bf16*)p.out)[row * p.ldo + c] = __float2bfloat16_rn(0.f);
  }
}

template <int NV8, int NM>
int launch(const evo_window_attn_params* p, cudaStream_t st) {
  const int dkp = (p->dk + 15) / 16 * 16;
  const int qst = NM * dkp + 8, kst = NM * dkp + 8, vst = NV8 * 8 + 8;
  // two K/V buffers (the next tile is fetched while the current one is in work) as long as two CTAs still fit an SM's shared memory
  const size_t tile = sizeof(bf16) * ((size_t)KT * kst + (size_t)KT * vst), qbytes = sizeof(bf16) * (size_t)WARPS * QROWS * qst;
  auto a16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
  const int vec = p->dk % 8 == 0 && p->dv % 8 == 0 && p->q_tok_stride % 8 == 0 && p->k_tok_stride % 8 == 0 && p->v_tok_stride % 8 == 0 &&
                  p->k_batch_stride % 8 == 0 && p->v_batch_stride % 8 == 0 && a16(p->q) && a16(p->k) && a16(p->v) &&
                  (p->pool <= 0 || (p->pool_tok_stride % 8 == 0 && p->pool_batch_stride % 8 == 0 && a16(p->pool_k) && a16(p->pool_v)));
  const int nbuf = vec && qbytes + 2 * tile <= 110 * 1024 ? 2 : 1;
  const size_t smem = qbytes + nbuf * tile;
  auto kern = window_attn_mma_kernel<NV8, NM>;
  if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int c8n = NM * dkp / 8;
  kern<<<dim3((unsigned)((p->Lq + WARPS * QROWS - 1) / (WARPS * QROWS)), p->H, p->B), WARPS * 32, smem, st>>>(*p, dkp, qst, kst, vst, vec,
                                                                                                                 make_int2(WARPS * 32 / c8n, WARPS * 32 % c8n), nbuf);
  return check_launch("evo_window_attn_fwd");
}

template <int NM>
int dispatch(const evo_window_attn_params* p, cudaStream_t st) {
  const int nv8 = (p->dv + 15) / 16 * 2;
  switch (nv8) {
    case 2: return launch<2, NM>(p, st);
    case 4: return launch<4, NM>(p, st);
    case 6: return launch<6, NM>(p, st);
    case 8: return launch<8, NM>(p, st);
    case 10: return launch<10, NM>(p, st);
    case 12: return launch<12, NM>(p, st);
    case 14: return launch<14, NM>(p, st);
    default: return launch<16, NM>(p, st);
  }
}

}  // namespace

int evo::window_attn_mma(const evo_window_attn_params* p, cudaStream_t st) {
  if (p->dtype != 0 || p->dk * p->n_maps > 256 || p->dk > 128 || p->dv > 128 || p->dv % 8 != 0 || p->Lq < 16) return 1;
  return p->n_maps == 2 ? dispatch<2>(p, st) : dispatch<1>(p, st);
}
