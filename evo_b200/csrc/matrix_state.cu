// Recurrences whose state is a (dk x dv) matrix per head, carried in fp32 registers for the whole call:
//   gated delta rule   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q        (evo_gated_delta_fwd)
//   state-space dual   S <- a S + (dt B) x^T;  y = S^T C + D x                             (evo_ssd_fwd)
//   matrix memory      m' = max(f + m, i);  S <- e^{f+m-m'} S + e^{i-m'} k v^T;  n alike;  o = S^T q / (max(|n.q|, e^{-m'}) + c)   (evo_mlstm_fwd)
// with everything around them that the recurrence consumes computed here in fp32 from the activated projections: the unit norms of
// q and k, sigmoid / softplus / exponentials of the per-head gates, and for the delta rule the head's RMS norm, weight and SiLU gate.
//
// One CTA per (head, sequence, group of value channels).  A thread owns CPT (two, when the registers allow) adjacent columns:
// every (key, query) pair read from shared memory then serves two columns, and the shared-memory pipe -- which bounded the
// one-column form at half its time -- sees half the traffic per multiply-add.  Column j of the state belongs to LPC adjacent lanes of one warp, each
// holding RPT rows in pairs (lane l, pair r: rows 2*(r*LPC + l) and + 1, so that the lanes of a column read consecutive 16-byte
// (key, query, key, query) entries of shared memory, without bank conflicts); column sums (S^T k, S^T q) are folded with shuffles, so the time loop has no
// barrier.  Value channels are independent in both recurrences: a head whose state does not fit one CTA's registers, or a call
// that would leave SMs idle, is spread over several CTAs by value channel; the delta rule's read-outs then go to an fp32
// workspace and a second small kernel applies the head norm, weight and gate.
// Prompts on so few (head, sequence) pairs that every CTA has an SM of its own put 16 lanes with half the rows on a column of 65 to 128 rows
// (twice the warps per SM for one more shuffle step per fold).
// TCH tokens are staged per round in shared memory: (k, q) pairs per state row, values, and the per-token numbers.
// The delta rule needs S^T k before it can write: both products are taken from the decayed state in one pass,
//   p = (gS)^T k,  r = (gS)^T q,  u = beta (v - p),  o = r + u (k . q),
// and the rank-one update follows with u -- one shuffle fold per token instead of two.
// The matrix memory's running maximum is a (max, +) scan over the round's tokens that one warp does between staging and the time loop.
// Its normaliser n (a vector per head) never enters the time loop: within a round n_t.q_t = P_t (n_0.q_t) + sum_{s<=t} (prod_{s<r<=t} a_r) b_s (k_s.q_t)
// with a, b the round's decay and input factors and P_t = a_0 .. a_t, so the warps take the round's k_s.q_t and n_0.q_t dot products from
// the staged rows (one thread per pair), one thread per token folds them, and n_0 is advanced to the round's end the same way; every CTA of a head does this
// for itself, so a head spread over several CTAs needs no exchange.
// The single-token step is the same kernel with L == 1.
#include "common.cuh"
#include <stdlib.h>
#include "../../include/evo_b200.h"
#include <math.h>
#include <algorithm>

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int TCH = 16;      // tokens staged per round
enum { MODE_DELTA = 0, MODE_SSD = 1, MODE_MLSTM = 2 };

// what both recurrences look like to the time loop
struct ScanArgs {
  const void* kk; const void* qq; const void* vv; int64_t ld;      // "key" (G*dk), "query" (G*dk), "value" (H*dv) columns of the activated rows
  const void* s0; const void* s1; int64_t lds;                     // per-head raw numbers: delta (b, a), ssd (dt, -)
  const void* A_log; const void* dt_bias; const void* Dskip;
  float unit_eps, q_scale;
  float* state; int zero_start;
  // delta epilogue
  const void* gate; int64_t ldg; const void* norm_w; float eps; void* out; int64_t ldo;
  // ssd output, or the un-normed read-outs of the other two when a head is spread over several CTAs: (rows, H*dv) fp32
  float* y;
  int B; int64_t L; int H, G, dk, dv;
  // matrix memory: gate biases, soft cap, running maximum (B, H), and beside y the reciprocal denominators per (row, head);
  // a head's state is its dk x dv matrix followed by the dk entries of the normaliser
  const void* i_bias; const void* f_bias; float cap, den_eps; float* mstate; float* em;
};

// soft cap c tanh(z / c) (c <= 0: none) and log sigmoid
__device__ __forceinline__ float soft_cap(float z, float c) { return c > 0.f ? c * tanhf(z / c) : z; }
__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int RPT, int LPC, int MODE>
__global__ void __launch_bounds__(RPT <= 4 ? 1024 : (RPT <= 32 ? 512 : 256), 1) matrix_state_kernel(ScanArgs p, int dvp) {
  constexpr int CPT = RPT <= 16 ? 2 : 1;                   // columns per thread
  extern __shared__ __align__(16) float smem[];
  const int dk = p.dk, dv = p.dv, dkp = LPC * RPT;
  float2* kq = reinterpret_cast<float2*>(smem);            // [TCH][dkp]   (key, query) per state row
  float* vs = smem + 2 * TCH * dkp;                        // [TCH][dvp]
  float* sc = vs + TCH * dvp;                              // [TCH][4]     delta: (g, beta, k.q, -)   ssd: (a, D, -, -)
  float* os = sc + TCH * 4;                                // [TCH][dvp]   delta / matrix-memory read-outs
  float* nvec = os + TCH * dvp;                            // [dkp]        matrix memory: the normaliser at the round's start
  float* kqd = nvec + dkp;                                 // [TCH][TCH]   k_s . q_t (s <= t)
  float* n0q = kqd + TCH * TCH;                            // [TCH]        n_0 . q_t
  const int h = blockIdx.x, b = blockIdx.y, g = h / (p.H / p.G);
  const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31, nw = nthr >> 5;
  const int j0 = blockIdx.z * dvp;                         // first value channel of this CTA
  const int jl = (tid / LPC) * CPT, l = tid % LPC, j = j0 + jl;      // first of the thread's columns, within the CTA and within the head
  const T* kp = (const T*)p.kk + (int64_t)g * dk;
  const T* qp = (const T*)p.qq + (int64_t)g * dk;
  const T* vp = (const T*)p.vv + (int64_t)h * dv;
  float* Sg = p.state ? p.state + ((int64_t)b * p.H + h) * dk * (int64_t)(MODE == MODE_MLSTM ? dv + 1 : dv) : nullptr;
  if (MODE == MODE_MLSTM)
    for (int e = tid; e < dkp; e += nthr) nvec[e] = (Sg && !p.zero_start && e < dk) ? Sg[(int64_t)dk * dv + e] : 0.f;
  const float A = MODE == MODE_MLSTM ? 0.f : expf(__bfloat162float(((const bf16*)p.A_log)[h]));
  const float dtb = MODE == MODE_MLSTM ? 0.f : __bfloat162float(((const bf16*)p.dt_bias)[h]);
  float mrun = (MODE == MODE_MLSTM && p.mstate && !p.zero_start) ? p.mstate[(int64_t)b * p.H + h] : 0.f;      // thread 0's: the running maximum
  const float Dh = MODE == MODE_SSD ? __bfloat162float(((const bf16*)p.Dskip)[h]) : 0.f;

  float S[CPT][RPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int k = 2 * ((r >> 1) * LPC + l) + (r & 1);
      S[c][r] = (Sg && !p.zero_start && j + c < dv && k < dk) ? Sg[(int64_t)k * dv + j + c] : 0.f;
    }

  for (int64_t t0 = 0; t0 < p.L; t0 += TCH) {
    const int nt = (int)min((int64_t)TCH, p.L - t0);
    const int64_t row0 = (int64_t)b * p.L + t0;
    __syncthreads();                                   // the previous round's staging and read-outs are no longer read
    // ---- staging: one warp per token
    for (int tt = warp; tt < nt; tt += nw) {
      const int64_t row = row0 + tt;
      if (MODE == MODE_DELTA) {
        float sk = 0.f, sq = 0.f, skq = 0.f;
        for (int e = lane; e < dk; e += 32) {
          const float kv = ldf(kp + row * p.ld + e), qv = ldf(qp + row * p.ld + e);
          sk = fmaf(kv, kv, sk); sq = fmaf(qv, qv, sq); skq = fmaf(kv, qv, skq);
        }
        sk = warp_sum(sk); sq = warp_sum(sq); skq = warp_sum(skq);
        const float rk = 1.0f / sqrtf(sk + p.unit_eps), rq = p.q_scale / sqrtf(sq + p.unit_eps);
        for (int e = lane; e < dkp; e += 32) {
          float2 o = make_float2(0.f, 0.f);
          if (e < dk) { o.x = ldf(kp + row * p.ld + e) * rk; o.y = ldf(qp + row * p.ld + e) * rq; }
          kq[tt * dkp + e] = o;
        }
        if (lane == 0) {
          const float bv = ldf((const T*)p.s0 + row * p.lds + h), av = ldf((const T*)p.s1 + row * p.lds + h);
          sc[tt * 4 + 0] = expf(-A * softplus_f(av + dtb));
          sc[tt * 4 + 1] = 1.f / (1.f + expf(-bv));
          sc[tt * 4 + 2] = skq * rk * rq;
        }
      } else if (MODE == MODE_MLSTM) {
        for (int e = lane; e < dkp; e += 32) {
          float2 o = make_float2(0.f, 0.f);
          if (e < dk) { o.x = ldf(kp + row * p.ld + e); o.y = ldf(qp + row * p.ld + e) * p.q_scale; }
          kq[tt * dkp + e] = o;
        }
        if (lane == 0) {                                  // log forget gate, log input gate; the scan below turns them into factors
          const float gi = ldf((const T*)p.s0 + row * p.lds + h) + __bfloat162float(((const bf16*)p.i_bias)[h]);
          const float gf = ldf((const T*)p.s1 + row * p.lds + h) + __bfloat162float(((const bf16*)p.f_bias)[h]);
          sc[tt * 4 + 0] = log_sigmoid(soft_cap(gf, p.cap));
          sc[tt * 4 + 1] = soft_cap(gi, p.cap);
        }
      } else {
        const float dt = softplus_f(ldf((const T*)p.s0 + row * p.lds + h) + dtb);
        for (int e = lane; e < dkp; e += 32) {
          float2 o = make_float2(0.f, 0.f);
          if (e < dk) { o.x = ldf(kp + row * p.ld + e) * dt; o.y = ldf(qp + row * p.ld + e); }
          kq[tt * dkp + e] = o;
        }
        if (lane == 0) { sc[tt * 4 + 0] = expf(-A * dt); sc[tt * 4 + 1] = Dh; }
      }
      for (int c = lane; c < dvp; c += 32) vs[tt * dvp + c] = j0 + c < dv ? ldf(vp + row * p.ld + j0 + c) : 0.f;
    }
    __syncthreads();
    if (MODE == MODE_MLSTM) {
      if (warp == 0) {
        // m_t = max(f_t + m_{t-1}, i_t) over the round as two prefix scans: with F_t = f_0 + .. + f_t,  m_t = F_t + max(m_start, max_{s<=t} (i_s - F_s))
        const bool on = lane < nt;
        const float f = on ? sc[lane * 4 + 0] : 0.f, i = on ? sc[lane * 4 + 1] : -INFINITY;
        float F = f;
#pragma unroll
        for (int o = 1; o < TCH; o <<= 1) { const float u = __shfl_up_sync(0xffffffffu, F, o); if (lane >= o) F += u; }
        float g = i - F;
#pragma unroll
        for (int o = 1; o < TCH; o <<= 1) { const float u = __shfl_up_sync(0xffffffffu, g, o); if (lane >= o) g = fmaxf(g, u); }
        const float m = F + fmaxf(mrun, g);
        float mprev = __shfl_up_sync(0xffffffffu, m, 1);
        if (lane == 0) mprev = mrun;
        if (on) { sc[lane * 4 + 0] = expf(f + mprev - m); sc[lane * 4 + 1] = expf(i - m); sc[lane * 4 + 2] = expf(-m); }
        mrun = __shfl_sync(0xffffffffu, m, nt - 1);
      }
      // the round's dot products, one thread each: pair (s, t), s <= t, has index t (t + 1) / 2 + s; after the pairs, n_0 . q_t.  Two state rows
      // (k, q, k, q) per 16-byte read; neighbouring threads hold neighbouring s (or, for n_0, t) and start that many reads into the row, so
      // that the threads of a quarter warp read different banks
      const int npair = nt * (nt + 1) / 2, nq4 = dkp / 2;
      for (int task = tid; task < npair + nt; task += nthr) {
        int t = task - npair, s_ = nt;
        if (task < npair) { t = 0; while ((t + 1) * (t + 2) / 2 <= task) ++t; s_ = task - t * (t + 1) / 2; }
        const float4* qt = reinterpret_cast<const float4*>(kq + t * dkp);
        float d0 = 0.f, d1 = 0.f;
        const int msk = nq4 - 1;                          // dkp is a power of two
        if (s_ < nt) {
          const float4* ks = reinterpret_cast<const float4*>(kq + s_ * dkp);
#pragma unroll 8
          for (int i = 0; i < nq4; ++i) { const int e = (s_ + i) & msk; const float4 a = ks[e], c = qt[e]; d0 = fmaf(a.x, c.y, d0); d1 = fmaf(a.z, c.w, d1); }
          kqd[s_ * TCH + t] = d0 + d1;
        } else {
          const float2* nv2 = reinterpret_cast<const float2*>(nvec);
#pragma unroll 8
          for (int i = 0; i < nq4; ++i) { const int e = (t + i) & msk; const float4 c = qt[e]; const float2 n2 = nv2[e]; d0 = fmaf(n2.x, c.y, d0); d1 = fmaf(n2.y, c.w, d1); }
          n0q[t] = d0 + d1;
        }
      }
      __syncthreads();
      // one thread per token folds its row of products into n_t . q_t and keeps the reciprocal denominator; the normaliser moves to the round's end
      if (tid < nt) {                                      // n_t . q_t = (..((n_0.q_t) a_0 + b_0 k_0.q_t) a_1 + ..) a_t + b_t k_t.q_t
        float acc = n0q[tid];
#pragma unroll
        for (int s_ = 0; s_ < TCH; ++s_)
          if (s_ <= tid) acc = fmaf(acc, sc[s_ * 4 + 0], sc[s_ * 4 + 1] * kqd[s_ * TCH + tid]);
        const float inv = 1.f / (fmaxf(fabsf(acc), sc[tid * 4 + 2]) + p.den_eps);
        sc[tid * 4 + 3] = inv;
        if (p.em && blockIdx.z == 0) p.em[(row0 + tid) * p.H + h] = inv;
      }
      for (int e = tid; e < dkp; e += nthr) {
        float n = nvec[e];
#pragma unroll
        for (int s_ = 0; s_ < TCH; ++s_)
          if (s_ < nt) n = fmaf(n, sc[s_ * 4 + 0], sc[s_ * 4 + 1] * kq[s_ * dkp + e].x);
        nvec[e] = n;
      }
    }
    // ---- time loop
    for (int tt = 0; tt < nt; ++tt) {
      float v[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) v[c] = vs[tt * dvp + jl + c];
      const float dec = sc[tt * 4 + 0];
      const float4* e = reinterpret_cast<const float4*>(kq + tt * dkp) + l;             // two state rows per 16-byte read; pair r at e[r * LPC]
      if (MODE == MODE_DELTA) {
        constexpr bool KEEP = RPT <= 16;                   // the keys stay in registers for the update, or are read again
        float pk[CPT], pq[CPT], kx[KEEP ? RPT : 2];
#pragma unroll
        for (int c = 0; c < CPT; ++c) pk[c] = pq[c] = 0.f;
#pragma unroll
        for (int r = 0; r < RPT / 2; ++r) {
          const float4 f = e[r * LPC];
          if (KEEP) { kx[2 * r] = f.x; kx[2 * r + 1] = f.z; }
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            S[c][2 * r] *= dec;          pk[c] = fmaf(S[c][2 * r], f.x, pk[c]);     pq[c] = fmaf(S[c][2 * r], f.y, pq[c]);
            S[c][2 * r + 1] *= dec;      pk[c] = fmaf(S[c][2 * r + 1], f.z, pk[c]); pq[c] = fmaf(S[c][2 * r + 1], f.w, pq[c]);
          }
        }
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1)
#pragma unroll
          for (int c = 0; c < CPT; ++c) { pk[c] += __shfl_xor_sync(0xffffffffu, pk[c], o); pq[c] += __shfl_xor_sync(0xffffffffu, pq[c], o); }
        const float beta = sc[tt * 4 + 1], kqd = sc[tt * 4 + 2];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          const float u = beta * (v[c] - pk[c]);
          if (KEEP) {
#pragma unroll
            for (int r = 0; r < RPT; ++r) S[c][r] = fmaf(kx[r], u, S[c][r]);
          } else {
#pragma unroll
            for (int r = 0; r < RPT / 2; ++r) {
              const float4 f = e[r * LPC];
              S[c][2 * r] = fmaf(f.x, u, S[c][2 * r]);
              S[c][2 * r + 1] = fmaf(f.z, u, S[c][2 * r + 1]);
            }
          }
          const float o = fmaf(u, kqd, pq[c]);
          if (l == 0) {
            if (p.y) { if (j + c < dv) p.y[((row0 + tt) * p.H + h) * dv + j + c] = o; }
            else os[tt * dvp + jl + c] = o;
          }
        }
      } else {
        float y[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) y[c] = 0.f;
        if (MODE == MODE_MLSTM) {
          const float inn = sc[tt * 4 + 1];
#pragma unroll
          for (int c = 0; c < CPT; ++c) v[c] *= inn;
        }
#pragma unroll
        for (int r = 0; r < RPT / 2; ++r) {
          const float4 f = e[r * LPC];
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            S[c][2 * r] = fmaf(dec, S[c][2 * r], f.x * v[c]);          y[c] = fmaf(S[c][2 * r], f.y, y[c]);
            S[c][2 * r + 1] = fmaf(dec, S[c][2 * r + 1], f.z * v[c]);  y[c] = fmaf(S[c][2 * r + 1], f.w, y[c]);
          }
        }
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1)
#pragma unroll
          for (int c = 0; c < CPT; ++c) y[c] += __shfl_xor_sync(0xffffffffu, y[c], o);
        if (MODE == MODE_MLSTM) {
#pragma unroll
          for (int c = 0; c < CPT; ++c)
            if (l == 0) {
              if (p.y) { if (j + c < dv) p.y[((row0 + tt) * p.H + h) * dv + j + c] = y[c]; }
              else os[tt * dvp + jl + c] = y[c];
            }
        } else {
          const float Dv = sc[tt * 4 + 1];
#pragma unroll
          for (int c = 0; c < CPT; ++c)
            if (l == 0 && j + c < dv) p.y[((row0 + tt) * p.H + h) * dv + j + c] = fmaf(Dv, v[c], y[c]);
        }
      }
    }
    if (MODE == MODE_MLSTM && !p.y) {
      __syncthreads();
      // normaliser, head norm, weight over all heads, sigmoid gate, store: one warp per token
      const bf16* nwt = (const bf16*)p.norm_w + (int64_t)h * dv;
      for (int tt = warp; tt < nt; tt += nw) {
        const int64_t row = row0 + tt;
        const float inv = sc[tt * 4 + 3];
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) { const float o = os[tt * dvp + c] * inv; ss = fmaf(o, o, ss); }
        ss = warp_sum(ss);
        const float rstd = inv / sqrtf(ss / (float)dv + p.eps);
        T* orow = (T*)p.out + row * p.ldo;
        const T* grow = (const T*)p.gate + row * p.ldg + (int64_t)h * dv;
        for (int c = lane; c < dv; c += 32)
          stf(orow + h * dv + c, os[tt * dvp + c] * rstd * __bfloat162float(nwt[c]) / (1.f + expf(-ldf(grow + c))));
        if (h == p.H - 1)
          for (int64_t c = (int64_t)p.H * dv + lane; c < p.ldo; c += 32) stf(orow + c, 0.f);
      }
    }
    if (MODE == MODE_DELTA && !p.y) {
      __syncthreads();
      // head norm, weight, SiLU gate, store: one warp per token
      const bf16* nwt = (const bf16*)p.norm_w;
      for (int tt = warp; tt < nt; tt += nw) {
        const int64_t row = row0 + tt;
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) { const float o = os[tt * dvp + c]; ss = fmaf(o, o, ss); }
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / (float)dv + p.eps);
        T* orow = (T*)p.out + row * p.ldo;
        const T* grow = (const T*)p.gate + row * p.ldg + (int64_t)h * dv;
        for (int c = lane; c < dv; c += 32) {
          const float gv = ldf(grow + c);
          stf(orow + h * dv + c, os[tt * dvp + c] * rstd * __bfloat162float(nwt[c]) * (gv / (1.f + expf(-gv))));
        }
        if (h == p.H - 1)
          for (int64_t c = (int64_t)p.H * dv + lane; c < p.ldo; c += 32) stf(orow + c, 0.f);
      }
    }
  }
  if (MODE == MODE_MLSTM && Sg && blockIdx.z == 0) {
    __syncthreads();                                     // the last round's normaliser is complete
    if (tid == 0) p.mstate[(int64_t)b * p.H + h] = mrun;
    for (int e = tid; e < dk; e += nthr) Sg[(int64_t)dk * dv + e] = nvec[e];
  }
  if (Sg) {
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int k = 2 * ((r >> 1) * LPC + l) + (r & 1);
        if (k < dk && j + c < dv) Sg[(int64_t)k * dv + j + c] = S[c][r];
      }
  }
}

// head norm, weight and SiLU gate of the delta rule's read-outs when a head was spread over several CTAs: one warp per (row, head)
template <typename T>
__global__ void __launch_bounds__(256) delta_head_norm_kernel(ScanArgs p) {
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (int64_t)p.B * p.L * p.H) return;
  const int64_t row = wid / p.H; const int h = (int)(wid % p.H);
  const float* r = p.y + wid * p.dv;
  float ss = 0.f;
  for (int c = lane; c < p.dv; c += 32) ss = fmaf(r[c], r[c], ss);
  ss = warp_sum(ss);
  const float rstd = 1.0f / sqrtf(ss / (float)p.dv + p.eps);
  T* orow = (T*)p.out + row * p.ldo;
  const T* grow = (const T*)p.gate + row * p.ldg + (int64_t)h * p.dv;
  const bf16* nw = (const bf16*)p.norm_w;
  for (int c = lane; c < p.dv; c += 32) {
    const float gv = ldf(grow + c);
    stf(orow + h * p.dv + c, r[c] * rstd * __bfloat162float(nw[c]) * (gv / (1.f + expf(-gv))));
  }
  if (h == p.H - 1)
    for (int64_t c = (int64_t)p.H * p.dv + lane; c < p.ldo; c += 32) stf(orow + c, 0.f);
}

// the same for the matrix memory's read-outs (rows, H, dv) with the reciprocal denominators beside them
template <typename T>
__global__ void __launch_bounds__(256) mlstm_head_norm_kernel(ScanArgs p) {
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (int64_t)p.B * p.L * p.H) return;
  const int64_t row = wid / p.H; const int h = (int)(wid % p.H);
  const int dv = p.dv;
  const float* r = p.y + wid * dv;
  const float inv = p.em[wid];
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) { const float o = r[c] * inv; ss = fmaf(o, o, ss); }
  ss = warp_sum(ss);
  const float rstd = inv / sqrtf(ss / (float)dv + p.eps);
  T* orow = (T*)p.out + row * p.ldo;
  const T* grow = (const T*)p.gate + row * p.ldg + (int64_t)h * dv;
  const bf16* nw = (const bf16*)p.norm_w + (int64_t)h * dv;
  for (int c = lane; c < dv; c += 32) stf(orow + h * dv + c, r[c] * rstd * __bfloat162float(nw[c]) / (1.f + expf(-ldf(grow + c))));
  if (h == p.H - 1)
    for (int64_t c = (int64_t)p.H * dv + lane; c < p.ldo; c += 32) stf(orow + c, 0.f);
}

struct Plan { int rpt, lpc, dvc, chunks; };
inline int thread_limit(int rpt) { return rpt <= 4 ? 1024 : (rpt <= 32 ? 512 : 256); }      // registers: rpt state rows per column per thread
inline int columns_per_thread(int rpt) { return rpt <= 16 ? 2 : 1; }
// about 8 lanes per column (three shuffle steps per fold), RPT = rows / lanes; the value channels a CTA takes follow from its
// thread limit, and long calls on few (head, sequence) pairs are spread further so that every SM has a CTA
inline Plan plan(int dk, int dv, int64_t ctas, int64_t L) {
  int rpt = 4;
  while (rpt < 64 && rpt * 8 < dk) rpt <<= 1;
  // prompts on so few (head, sequence) pairs that every CTA of 512 threads gets an SM of its own: 16 lanes per column with half the rows
  // each (one more shuffle step per fold) put twice the warps on an SM.  EVO_B200_MATRIX_STATE_LANES = 8 | 16 fixes the choice (comparisons).
  static const int forced = [] { const char* e = getenv("EVO_B200_MATRIX_STATE_LANES"); return e ? atoi(e) : 0; }();
  if (rpt == 16 && L >= 256 && forced != 8 && (forced == 16 || ctas * ((dv + 63) / 64) <= device_sm_count())) rpt = 8;
  int lpc = 1;
  while (lpc * rpt < dk) lpc <<= 1;
  if (lpc > 32) return {0, 0, 0, 0};
  const int cpt = columns_per_thread(rpt);
  const int gran = std::max(cpt, 32 * cpt / lpc);                    // columns of one warp: a CTA takes whole warps
  const int dvp = (dv + gran - 1) / gran * gran;
  const int per_cta = thread_limit(rpt) / 32 * gran;
  int chunks = (dvp + per_cta - 1) / per_cta;
  if (L >= 256)
    while (ctas * chunks < device_sm_count() && (dvp / gran + 2 * chunks - 1) / (2 * chunks) * gran >= 64 && 2 * chunks <= dvp / gran) chunks *= 2;   // a CTA keeps >= 64 columns: each one stages the head's keys and queries again
  const int dvc = (dvp / gran + chunks - 1) / chunks * gran;
  return {rpt, lpc, dvc, (dv + dvc - 1) / dvc};
}

template <typename T, int RPT, int LPC, int MODE>
int launch(const ScanArgs& a, const Plan& pl, cudaStream_t st, const char* what) {
  const size_t smem = sizeof(float) * ((size_t)2 * TCH * LPC * RPT + (size_t)2 * TCH * pl.dvc + (size_t)TCH * 4 + (size_t)LPC * RPT + (size_t)TCH * TCH + TCH);
  auto kern = matrix_state_kernel<T, RPT, LPC, MODE>;
  if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3(a.H, a.B, pl.chunks), dim3(LPC * pl.dvc / columns_per_thread(RPT)), smem, st>>>(a, pl.dvc);
  int rc = check_launch(what);
  if (rc || MODE == MODE_SSD || !a.y) return rc;
  const int64_t warps = (int64_t)a.B * a.L * a.H;
  if (MODE == MODE_DELTA) delta_head_norm_kernel<T><<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(a);
  else mlstm_head_norm_kernel<T><<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(a);
  return check_launch(what);
}

template <typename T, int MODE>
int dispatch(ScanArgs a, void* workspace, size_t workspace_bytes, cudaStream_t st, const char* what) {
  const Plan pl = plan(a.dk, a.dv, (int64_t)a.B * a.H, a.L);
  if (pl.rpt == 0) { set_error("%s: a state of %d rows per head does not fit (rows <= 2048)", what, a.dk); return -1; }
  if (MODE != MODE_SSD && pl.chunks > 1) {
    const size_t rows = (size_t)a.B * a.L * a.H;
    const size_t need = sizeof(float) * rows * (a.dv + (MODE == MODE_MLSTM ? 1 : 0));
    if (!workspace || workspace_bytes < need) { set_error("%s: workspace too small (%zu < %zu)", what, workspace_bytes, need); return -1; }
    a.y = (float*)workspace;
    if (MODE == MODE_MLSTM) a.em = a.y + rows * a.dv;
  }
  // the (rows per lane, lanes per column) pairs plan() can return: both are compile-time constants of the time loop
  switch (pl.rpt * 100 + pl.lpc) {
    case 401: return launch<T, 4, 1, MODE>(a, pl, st, what);
    case 402: return launch<T, 4, 2, MODE>(a, pl, st, what);
    case 404: return launch<T, 4, 4, MODE>(a, pl, st, what);
    case 408: return launch<T, 4, 8, MODE>(a, pl, st, what);
    case 808: return launch<T, 8, 8, MODE>(a, pl, st, what);
    case 816: return launch<T, 8, 16, MODE>(a, pl, st, what);
    case 1608: return launch<T, 16, 8, MODE>(a, pl, st, what);
    case 3208: return launch<T, 32, 8, MODE>(a, pl, st, what);
    case 6408: return launch<T, 64, 8, MODE>(a, pl, st, what);
    case 6416: return launch<T, 64, 16, MODE>(a, pl, st, what);
    case 6432: return launch<T, 64, 32, MODE>(a, pl, st, what);
  }
  set_error("%s: no kernel for %d rows per lane x %d lanes", what, pl.rpt, pl.lpc);
  return -1;
}

}  // namespace

extern "C" size_t evo_gated_delta_workspace(const evo_gated_delta_params* p) {
  const Plan pl = plan(p->dk, p->dv, (int64_t)p->B * p->H, p->L);
  return pl.chunks > 1 ? sizeof(float) * (size_t)p->B * p->L * p->H * p->dv : 0;
}

extern "C" int evo_gated_delta_fwd(const evo_gated_delta_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  EVO_REQUIRE(p->q && p->k && p->v && p->b && p->a && p->gate && p->A_log && p->dt_bias && p->norm_w && p->out, "evo_gated_delta_fwd: null argument");
  EVO_REQUIRE(p->B >= 0 && p->L >= 0 && p->H > 0 && p->G > 0 && p->H % p->G == 0 && p->dk > 0 && p->dv > 0 && p->ldo >= (int64_t)p->H * p->dv,
              "evo_gated_delta_fwd: bad shape");
  if (p->B == 0 || p->L == 0) return 0;
  ScanArgs a = {};
  a.kk = p->k; a.qq = p->q; a.vv = p->v; a.ld = p->ld;
  a.s0 = p->b; a.s1 = p->a; a.lds = p->ldz;
  a.A_log = p->A_log; a.dt_bias = p->dt_bias;
  a.unit_eps = p->unit_eps; a.q_scale = p->q_scale;
  a.state = p->state; a.zero_start = p->zero_start;
  a.gate = p->gate; a.ldg = p->ldz; a.norm_w = p->norm_w; a.eps = p->eps; a.out = p->out; a.ldo = p->ldo;
  a.B = p->B; a.L = p->L; a.H = p->H; a.G = p->G; a.dk = p->dk; a.dv = p->dv;
  return p->dtype ? dispatch<float, MODE_DELTA>(a, workspace, workspace_bytes, (cudaStream_t)stream, "evo_gated_delta_fwd")
                  : dispatch<bf16, MODE_DELTA>(a, workspace, workspace_bytes, (cudaStream_t)stream, "evo_gated_delta_fwd");
}

extern "C" int evo_ssd_fwd(const evo_ssd_params* p, void* stream) {
  EVO_REQUIRE(p->x && p->Bm && p->Cm && p->dt && p->A_log && p->dt_bias && p->D && p->y, "evo_ssd_fwd: null argument");
  EVO_REQUIRE(p->B >= 0 && p->L >= 0 && p->H > 0 && p->G > 0 && p->H % p->G == 0 && p->N > 0 && p->dv > 0, "evo_ssd_fwd: bad shape");
  if (p->B == 0 || p->L == 0) return 0;
  ScanArgs a = {};
  a.kk = p->Bm; a.qq = p->Cm; a.vv = p->x; a.ld = p->ld;
  a.s0 = p->dt; a.lds = p->ld_dt;
  a.A_log = p->A_log; a.dt_bias = p->dt_bias; a.Dskip = p->D;
  a.state = p->state; a.zero_start = p->zero_start;
  a.y = p->y;
  a.B = p->B; a.L = p->L; a.H = p->H; a.G = p->G; a.dk = p->N; a.dv = p->dv;
  return p->dtype ? dispatch<float, MODE_SSD>(a, nullptr, 0, (cudaStream_t)stream, "evo_ssd_fwd") : dispatch<bf16, MODE_SSD>(a, nullptr, 0, (cudaStream_t)stream, "evo_ssd_fwd");
}

namespace {
inline ScanArgs mlstm_args(const evo_mlstm_params* p) {
  ScanArgs a = {};
  a.kk = p->k; a.qq = p->q; a.vv = p->v; a.ld = p->ld;
  a.s0 = p->gi; a.s1 = p->gf; a.lds = p->ldg;
  a.i_bias = p->i_bias; a.f_bias = p->f_bias; a.cap = p->cap; a.den_eps = p->den_eps; a.q_scale = p->q_scale;
  a.state = p->state; a.mstate = p->mstate; a.zero_start = p->zero_start;
  a.gate = p->gate; a.ldg = p->ld_gate; a.norm_w = p->norm_w; a.eps = p->eps; a.out = p->out; a.ldo = p->ldo;
  a.B = p->B; a.L = p->L; a.H = p->H; a.G = p->H; a.dk = p->dk; a.dv = p->dv;
  return a;
}
}  // namespace

extern "C" size_t evo_mlstm_workspace(const evo_mlstm_params* p) {
  const Plan pl = plan(p->dk, p->dv, (int64_t)p->B * p->H, p->L);
  return pl.chunks > 1 ? sizeof(float) * (size_t)p->B * p->L * p->H * (p->dv + 1) : 0;
}

extern "C" int evo_mlstm_fwd(const evo_mlstm_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  EVO_REQUIRE(p->q && p->k && p->v && p->gi && p->gf && p->i_bias && p->f_bias && p->gate && p->norm_w && p->out, "evo_mlstm_fwd: null argument");
  EVO_REQUIRE((p->state == nullptr) == (p->mstate == nullptr), "evo_mlstm_fwd: the matrix state and the running maximum come together");
  EVO_REQUIRE(p->B >= 0 && p->L >= 0 && p->H > 0 && p->dk > 0 && p->dv > 0 && p->ldo >= (int64_t)p->H * p->dv, "evo_mlstm_fwd: bad shape");
  if (p->B == 0 || p->L == 0) return 0;
  const ScanArgs a = mlstm_args(p);
  return p->dtype ? dispatch<float, MODE_MLSTM>(a, workspace, workspace_bytes, (cudaStream_t)stream, "evo_mlstm_fwd")
                  : dispatch<bf16, MODE_MLSTM>(a, workspace, workspace_bytes, (cudaStream_t)stream, "evo_mlstm_fwd");
}
