// Matrix-memory recurrent layer (the mLSTM cell of xLSTM, stabilised form) for a ragged step.
//
// Per head, with q scaled by D^-1/2, log input gate i_t and log forget gate f_t (both soft-capped), state
// (S [D, V], n [D], m) that starts at (0, 0, 0):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T        n_t likewise with k_t alone
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// The state is fp32 and lives in a per-sequence SLOT between steps; an entry whose first position is 0 starts
// from zero whatever the slot held.  Gates, decays, the state update and the read-out are fp32; q, k, v and the
// gate pre-activations come from a packed projection row of element type E.
//
// mlstm_scan_kernel walks the rows of one entry in order (one CTA per entry, head and 32-column slice of V: the
// columns of S are independent, n and m are recomputed by every slice).  mlstm_out_kernel then divides each head's
// output by its root mean square, applies the per-channel weight and the sigmoid output gate.
#include <math.h>

#include "common.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float m_to_f(E v);
template <> __device__ __forceinline__ float m_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float m_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E m_from_f(float v);
template <> __device__ __forceinline__ float m_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 m_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

struct MlstmArgs {
  const int32_t* ent;
  int H, D, V;
  int ldp, q_off, k_off, v_off, i_off, f_off;
  const float* i_bias;  // [H]
  const float* f_bias;
  float cap;            // soft cap of the gate pre-activations, <= 0: none
  float* S;             // [slots, H, D, V]
  float* n;             // [slots, H, D]
  float* m;             // [slots, H]
};

constexpr int kMlCols = 32, kMlGroups = 8, kMlThreads = kMlCols * kMlGroups;

__device__ __forceinline__ float soft_cap(float x, float cap) { return cap > 0.f ? cap * tanhf(x / cap) : x; }
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename E>
__global__ void __launch_bounds__(kMlThreads)
mlstm_scan_kernel(const E* __restrict__ proj, float* __restrict__ o, MlstmArgs a) {
  extern __shared__ float sm[];
  float* S = sm;                         // [D][kMlCols]
  float* qs = S + (size_t)a.D * kMlCols;  // [D]
  float* ks = qs + a.D;                  // [D]
  float* ns = ks + a.D;                  // [D]
  float* red = ns + a.D;                 // [kMlGroups][kMlCols]
  float* rnq = red + kMlThreads;         // [kMlGroups]
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(a.ent)[blockIdx.x];  // slot, row0, n, start
  const int h = blockIdx.y, c0 = blockIdx.z * kMlCols;
  const int tid = threadIdx.x, col = tid % kMlCols, grp = tid / kMlCols;
  const int c = c0 + col;
  const bool col_ok = c < a.V;
  const bool fresh = e.w == 0;
  float* Sg = a.S + ((size_t)e.x * a.H + h) * a.D * a.V;
  float* ng = a.n + ((size_t)e.x * a.H + h) * a.D;
  float* mg = a.m + (size_t)e.x * a.H + h;
  for (int d = grp; d < a.D; d += kMlGroups) S[d * kMlCols + col] = (fresh || !col_ok) ? 0.f : Sg[(size_t)d * a.V + c];
  for (int d = tid; d < a.D; d += kMlThreads) ns[d] = fresh ? 0.f : ng[d];
  float m = fresh ? 0.f : *mg;
  const float qscale = 1.f / sqrtf((float)a.D);
  const float ib = a.i_bias ? a.i_bias[h] : 0.f, fb = a.f_bias ? a.f_bias[h] : 0.f;
  __syncthreads();
  for (int t = 0; t < e.z; ++t) {
    const int row = e.y + t;
    const E* pr = proj + (size_t)row * a.ldp;
    for (int d = tid; d < a.D; d += kMlThreads) {
      qs[d] = m_to_f(pr[a.q_off + h * a.D + d]) * qscale;
      ks[d] = m_to_f(pr[a.k_off + h * a.D + d]);
    }
    const float v = col_ok ? m_to_f(pr[a.v_off + h * a.V + c]) : 0.f;
    const float ig = soft_cap(m_to_f(pr[a.i_off + h]) + ib, a.cap);
    const float fg = log_sigmoid(soft_cap(m_to_f(pr[a.f_off + h]) + fb, a.cap));
    const float m_new = fmaxf(fg + m, ig);
    const float da = expf(fg + m - m_new), db = expf(ig - m_new);
    __syncthreads();
    float num = 0.f, nq = 0.f;
    for (int d = grp; d < a.D; d += kMlGroups) {
      const float kd = ks[d], qd = qs[d];
      const float s = da * S[d * kMlCols + col] + db * kd * v;
      S[d * kMlCols + col] = s;
      num = fmaf(s, qd, num);
      if (col == 0) {
        const float nn = da * ns[d] + db * kd;
        ns[d] = nn;
        nq = fmaf(nn, qd, nq);
      }
    }
    red[grp * kMlCols + col] = num;
    if (col == 0) rnq[grp] = nq;
    __syncthreads();
    if (tid < kMlCols && col_ok) {
      float s = 0.f, q = 0.f;
#pragma unroll
      for (int g = 0; g < kMlGroups; ++g) { s += red[g * kMlCols + tid]; q += rnq[g]; }
      const float den = fmaxf(fabsf(q), expf(-m_new)) + 1e-6f;
      o[((size_t)row * a.H + h) * a.V + c] = s / den;
    }
    m = m_new;
    __syncthreads();
  }
  if (col_ok)
    for (int d = grp; d < a.D; d += kMlGroups) Sg[(size_t)d * a.V + c] = S[d * kMlCols + col];
  if (blockIdx.z == 0) {
    for (int d = tid; d < a.D; d += kMlThreads) ng[d] = ns[d];
    if (tid == 0) *mg = m;
  }
}

// ---- portions of prompts: the same recurrence, 64 positions at a time ------------------------------------------
// Within a block of L positions (t = 1..L) let b_t be the running sum of the log forget gates, a_s = i_s - b_s and
// M_t = max(m_0, max_{s<=t} a_s).  Unrolling the recurrence gives m_t = b_t + M_t and
//     S_t = e^{m_0 - M_t} S_0 + sum_{s<=t} e^{a_s - M_t} k_s v_s^T          (n_t likewise)
// so the read-outs of the whole block are two small matrix products, (Q K^T masked and weighted by e^{a_s - M_t}) V
// plus e^{m_0 - M_t} Q S_0, and the state moves once per block: S_L = e^{m_0 - M_L} S_0 + K^T diag(e^{a_s - M_L}) V.
// Every exponent is <= 0.  All of it fp32 on the CUDA cores (the state and what enters it stay in 32-bit).
// One CTA per (entry, head, 64-column slice of V); q and k of the block are held transposed in shared memory.
constexpr int kMcL = 64, kMcLp = 68, kMcCols = 64, kMcThreads = 256;

template <typename E>
__global__ void __launch_bounds__(kMcThreads)
mlstm_chunk_kernel(const E* __restrict__ proj, float* __restrict__ o, MlstmArgs a) {
  extern __shared__ __align__(16) float smc[];
  const int D = a.D;
  float* qT = smc;                          // [D][kMcLp]
  float* kT = qT + (size_t)D * kMcLp;       // [D][kMcLp]
  float* Ss = kT + (size_t)D * kMcLp;       // [D][kMcCols]
  float* AT = Ss + (size_t)D * kMcCols;     // [L][kMcLp]   AT[s][t]
  float* vs = AT + kMcL * kMcLp;            // [L][kMcCols]
  float* ns = vs + kMcL * kMcCols;          // [D]
  float* av = ns + D;                       // [L] a_s
  float* Mv = av + kMcL;                    // [L] M_t
  float* bv = Mv + kMcL;                    // [L] b_t
  float* qn = bv + kMcL;                    // [L] n . q per row
  float* us = qn + kMcL;                    // [L] e^{a_s - M_L}
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(a.ent)[blockIdx.x];
  const int h = blockIdx.y, c0 = blockIdx.z * kMcCols;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const bool fresh = e.w == 0;
  float* Sg = a.S + ((size_t)e.x * a.H + h) * D * a.V;
  float* ng = a.n + ((size_t)e.x * a.H + h) * D;
  float* mg = a.m + (size_t)e.x * a.H + h;
  for (int i = tid; i < D * kMcCols; i += kMcThreads) {
    const int d = i / kMcCols, c = c0 + i % kMcCols;
    Ss[i] = (fresh || c >= a.V) ? 0.f : Sg[(size_t)d * a.V + c];
  }
  for (int d = tid; d < D; d += kMcThreads) ns[d] = fresh ? 0.f : ng[d];
  float m0 = fresh ? 0.f : *mg;
  const float qscale = 1.f / sqrtf((float)D);
  const float ib = a.i_bias ? a.i_bias[h] : 0.f, fb = a.f_bias ? a.f_bias[h] : 0.f;
  __syncthreads();

  for (int t0 = 0; t0 < e.z; t0 += kMcL) {
    const int len = min(kMcL, e.z - t0);
    const E* base = proj + (size_t)(e.y + t0) * a.ldp;
    // q, k transposed (zero beyond len), v slice, gates
    if (sizeof(E) == 2 && D % 8 == 0 && (a.q_off + h * D) % 8 == 0 && (a.k_off + h * D) % 8 == 0 && a.ldp % 8 == 0) {
      // 16-byte loads; consecutive threads take consecutive rows so that the transposed stores do not collide
#pragma unroll 4
      for (int i = tid; i < kMcL * (D / 8); i += kMcThreads) {
        const int t = i % kMcL, d8 = i / kMcL;
        uint4 uq = make_uint4(0, 0, 0, 0), uk = uq;
        if (t < len) {
          uq = ld_16B(base + (size_t)t * a.ldp + a.q_off + h * D + d8 * 8);
          uk = ld_16B(base + (size_t)t * a.ldp + a.k_off + h * D + d8 * 8);
        }
        float fq[8], fk[8];
        unpack8(uq, fq);
        unpack8(uk, fk);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          qT[(d8 * 8 + j) * kMcLp + t] = fq[j] * qscale;
          kT[(d8 * 8 + j) * kMcLp + t] = fk[j];
        }
      }
    } else {
      for (int i = tid; i < kMcL * D; i += kMcThreads) {
        const int t = i / D, d = i - t * D;
        float qv = 0.f, kv = 0.f;
        if (t < len) {
          qv = m_to_f(base[(size_t)t * a.ldp + a.q_off + h * D + d]) * qscale;
          kv = m_to_f(base[(size_t)t * a.ldp + a.k_off + h * D + d]);
        }
        qT[d * kMcLp + t] = qv;
        kT[d * kMcLp + t] = kv;
      }
    }
    for (int i = tid; i < kMcL * kMcCols; i += kMcThreads) {
      const int t = i / kMcCols, c = c0 + i % kMcCols;
      vs[i] = (t < len && c < a.V) ? m_to_f(base[(size_t)t * a.ldp + a.v_off + h * a.V + c]) : 0.f;
    }
    if (tid < kMcL) {
      float ig = -INFINITY, fg = 0.f;
      if (tid < len) {
        ig = soft_cap(m_to_f(base[(size_t)tid * a.ldp + a.i_off + h]) + ib, a.cap);
        fg = log_sigmoid(soft_cap(m_to_f(base[(size_t)tid * a.ldp + a.f_off + h]) + fb, a.cap));
      }
      av[tid] = ig;   // for now: i_s
      bv[tid] = fg;   // for now: f_s
    }
    __syncthreads();
    if (tid < 32) {  // running sums and maxima over the block: two positions per lane, warp scans between the lanes
      const float f0 = bv[2 * tid], f1 = bv[2 * tid + 1];
      float run = f0 + f1;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, run, o);
        if (tid >= o) run += up;
      }
      const float b1 = run, b0 = run - f1;           // inclusive sums at 2*lane and 2*lane + 1
      const float a0 = av[2 * tid] - b0, a1 = av[2 * tid + 1] - b1;
      float mx = fmaxf(a0, a1);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, mx, o);
        if (tid >= o) mx = fmaxf(mx, up);
      }
      const float before = __shfl_up_sync(0xffffffffu, mx, 1);
      const float M0 = fmaxf(m0, fmaxf(tid > 0 ? before : -INFINITY, a0));
      bv[2 * tid] = b0; bv[2 * tid + 1] = b1;
      av[2 * tid] = a0; av[2 * tid + 1] = a1;
      Mv[2 * tid] = M0; Mv[2 * tid + 1] = fmaxf(M0, a1);
    }
    __syncthreads();
    if (tid < kMcL) us[tid] = expf(av[tid] - Mv[kMcL - 1]);  // weights of the block's inputs in the state at its end
    // AT[s][t] = (q_t . k_s) e^{a_s - M_t} for s <= t, else 0: rows t = 4ty.., columns s = 4tx..
    {
      float acc[4][4] = {};
#pragma unroll 4
      for (int d = 0; d < D; ++d) {
        const float4 qa = *reinterpret_cast<const float4*>(qT + d * kMcLp + 4 * ty);
        const float4 kb = *reinterpret_cast<const float4*>(kT + d * kMcLp + 4 * tx);
        const float qv[4] = {qa.x, qa.y, qa.z, qa.w}, kv[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int t = 4 * ty + i, sidx = 4 * tx + j;
          AT[sidx * kMcLp + t] = (sidx <= t) ? acc[i][j] * expf(av[sidx] - Mv[t]) : 0.f;
        }
    }
    // n . q of the incoming state, per row
    if (tid < kMcL) {
      float d0 = 0.f, d1 = 0.f;
      int d = 0;
      for (; d + 1 < D; d += 2) {
        d0 = fmaf(ns[d], qT[d * kMcLp + tid], d0);
        d1 = fmaf(ns[d + 1], qT[(d + 1) * kMcLp + tid], d1);
      }
      if (d < D) d0 = fmaf(ns[d], qT[d * kMcLp + tid], d0);
      qn[tid] = d0 + d1;
    }
    __syncthreads();
    // read-out: rows t = 4ty.., columns c = 4tx..
    {
      float inter[4][4] = {}, intra[4][4] = {};
#pragma unroll 4
      for (int d = 0; d < D; ++d) {
        const float4 qa = *reinterpret_cast<const float4*>(qT + d * kMcLp + 4 * ty);
        const float4 sb = *reinterpret_cast<const float4*>(Ss + d * kMcCols + 4 * tx);
        const float qv[4] = {qa.x, qa.y, qa.z, qa.w}, sv[4] = {sb.x, sb.y, sb.z, sb.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) inter[i][j] = fmaf(qv[i], sv[j], inter[i][j]);
      }
      float rowsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int sidx = 0; sidx < len; ++sidx) {
        const float4 aa = *reinterpret_cast<const float4*>(AT + sidx * kMcLp + 4 * ty);
        const float4 vb = *reinterpret_cast<const float4*>(vs + sidx * kMcCols + 4 * tx);
        const float aw[4] = {aa.x, aa.y, aa.z, aa.w}, vv[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          rowsum[i] += aw[i];
#pragma unroll
          for (int j = 0; j < 4; ++j) intra[i][j] = fmaf(aw[i], vv[j], intra[i][j]);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = 4 * ty + i;
        if (t >= len) continue;
        const float g = expf(m0 - Mv[t]);
        const float den = fmaxf(fabsf(g * qn[t] + rowsum[i]), expf(-(bv[t] + Mv[t]))) + 1e-6f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + 4 * tx + j;
          if (c < a.V) o[((size_t)(e.y + t0 + t) * a.H + h) * a.V + c] = (g * inter[i][j] + intra[i][j]) / den;
        }
      }
    }
    __syncthreads();
    // the state moves to the end of the block
    {
      const float ML = Mv[kMcL - 1], gL = expf(m0 - ML);
      // 8 rows x 4 columns per thread and pass: one value row and one weight per position serve 32 FMAs
      for (int dbase = 0; dbase < D; dbase += 128) {
        float acc[8][4] = {};
        float nacc[8] = {};
        for (int sidx = 0; sidx < len; ++sidx) {
          const float u = us[sidx];
          const float4 vb = *reinterpret_cast<const float4*>(vs + sidx * kMcCols + 4 * tx);
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int d = dbase + ty + 16 * r;
            const float uk = d < D ? u * kT[d * kMcLp + sidx] : 0.f;
            acc[r][0] = fmaf(uk, vb.x, acc[r][0]); acc[r][1] = fmaf(uk, vb.y, acc[r][1]);
            acc[r][2] = fmaf(uk, vb.z, acc[r][2]); acc[r][3] = fmaf(uk, vb.w, acc[r][3]);
            nacc[r] += uk;
          }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int d = dbase + ty + 16 * r;
          if (d >= D) continue;
          float4* sp = reinterpret_cast<float4*>(Ss + d * kMcCols + 4 * tx);
          float4 sv = *sp;
          sv.x = gL * sv.x + acc[r][0]; sv.y = gL * sv.y + acc[r][1];
          sv.z = gL * sv.z + acc[r][2]; sv.w = gL * sv.w + acc[r][3];
          *sp = sv;
          if (tx == 0) ns[d] = gL * ns[d] + nacc[r];
        }
      }
      m0 = bv[kMcL - 1] + ML;
    }
    __syncthreads();
  }
  for (int i = tid; i < D * kMcCols; i += kMcThreads) {
    const int d = i / kMcCols, c = c0 + i % kMcCols;
    if (c < a.V) Sg[(size_t)d * a.V + c] = Ss[i];
  }
  if (blockIdx.z == 0) {
    for (int d = tid; d < D; d += kMcThreads) ng[d] = ns[d];
    if (tid == 0) *mg = m0;
  }
}

// ---- long portions: the blocks of one sequence in parallel ------------------------------------------------------
// The block form above walks a sequence's blocks in order inside one CTA, which leaves most SMs idle for a single long
// prompt.  Here every 64-position block gets its own CTAs, in three passes over tiles[2c] = entry, tiles[2c+1] = first
// row of block c within the entry (the blocks of an entry are consecutive):
//   pass 1 (parallel):  what block c adds to the state, as if it started from nothing: with A_c = max_s a_s,
//                       U_c = sum_s e^{a_s - A_c} k_s v_s^T, nU_c likewise, and the scalars (b_L, A_c);
//   pass 2 (in order, elementwise): S_in(c) is stored where U_c was, then S <- e^{m_0 - M} S + e^{A_c - M} U_c with
//                       M = max(m_0, A_c), m_0 <- b_L + M; the sequence's slot gets the final state;
//   pass 3 (parallel):  the read-outs of block c from (S_in(c), n_in(c), m_0(c)) as in the block form.
struct MlstmPar {
  const int32_t* tiles;
  float* cS;   // [blocks, H, D, V]
  float* cn;   // [blocks, H, D]
  float* csc;  // [blocks, H, 4] = (b_L, A_c, m_0 of the block, -)
};

template <typename E>
__device__ __forceinline__ void mlstm_load_kv_gates(const E* base, const MlstmArgs& a, int h, int len, int c0, float qscale,
                                                    float ib, float fb, float* qT, float* kT, float* vs, float* av,
                                                    float* bv, bool want_q) {
  const int D = a.D, tid = threadIdx.x;
  if (sizeof(E) == 2 && D % 8 == 0 && (a.q_off + h * D) % 8 == 0 && (a.k_off + h * D) % 8 == 0 && a.ldp % 8 == 0) {
#pragma unroll 4
    for (int i = tid; i < kMcL * (D / 8); i += kMcThreads) {
      const int t = i % kMcL, d8 = i / kMcL;
      uint4 uq = make_uint4(0, 0, 0, 0), uk = uq;
      if (t < len) {
        if (want_q) uq = ld_16B(base + (size_t)t * a.ldp + a.q_off + h * D + d8 * 8);
        uk = ld_16B(base + (size_t)t * a.ldp + a.k_off + h * D + d8 * 8);
      }
      float fq[8], fk[8];
      unpack8(uq, fq);
      unpack8(uk, fk);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (want_q) qT[(d8 * 8 + j) * kMcLp + t] = fq[j] * qscale;
        kT[(d8 * 8 + j) * kMcLp + t] = fk[j];
      }
    }
  } else {
    for (int i = tid; i < kMcL * D; i += kMcThreads) {
      const int t = i / D, d = i - t * D;
      float qv = 0.f, kv = 0.f;
      if (t < len) {
        if (want_q) qv = m_to_f(base[(size_t)t * a.ldp + a.q_off + h * D + d]) * qscale;
        kv = m_to_f(base[(size_t)t * a.ldp + a.k_off + h * D + d]);
      }
      if (want_q) qT[d * kMcLp + t] = qv;
      kT[d * kMcLp + t] = kv;
    }
  }
  for (int i = tid; i < kMcL * kMcCols; i += kMcThreads) {
    const int t = i / kMcCols, c = c0 + i % kMcCols;
    vs[i] = (t < len && c < a.V) ? m_to_f(base[(size_t)t * a.ldp + a.v_off + h * a.V + c]) : 0.f;
  }
  if (tid < kMcL) {
    float ig = -INFINITY, fg = 0.f;
    if (tid < len) {
      ig = soft_cap(m_to_f(base[(size_t)tid * a.ldp + a.i_off + h]) + ib, a.cap);
      fg = log_sigmoid(soft_cap(m_to_f(base[(size_t)tid * a.ldp + a.f_off + h]) + fb, a.cap));
    }
    av[tid] = ig;
    bv[tid] = fg;
  }
}

// Warp 0: b_t (running sum of the log forget gates), a_s = i_s - b_s and M_t = max(m_start, max_{s<=t} a_s).
__device__ __forceinline__ void mlstm_block_scan(float m_start, float* av, float* bv, float* Mv) {
  const int tid = threadIdx.x;
  if (tid < 32) {
    const float f0 = bv[2 * tid], f1 = bv[2 * tid + 1];
    float run = f0 + f1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, run, o);
      if (tid >= o) run += up;
    }
    const float b1 = run, b0 = run - f1;
    const float a0 = av[2 * tid] - b0, a1 = av[2 * tid + 1] - b1;
    float mx = fmaxf(a0, a1);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, mx, o);
      if (tid >= o) mx = fmaxf(mx, up);
    }
    const float before = __shfl_up_sync(0xffffffffu, mx, 1);
    const float M0 = fmaxf(m_start, fmaxf(tid > 0 ? before : -INFINITY, a0));
    bv[2 * tid] = b0; bv[2 * tid + 1] = b1;
    av[2 * tid] = a0; av[2 * tid + 1] = a1;
    Mv[2 * tid] = M0; Mv[2 * tid + 1] = fmaxf(M0, a1);
  }
}

template <typename E>
__global__ void __launch_bounds__(kMcThreads)
mlstm_par_local_kernel(const E* __restrict__ proj, MlstmArgs a, MlstmPar p) {
  extern __shared__ __align__(16) float smc[];
  const int D = a.D;
  float* kT = smc;                          // [D][kMcLp]
  float* vs = kT + (size_t)D * kMcLp;       // [L][kMcCols]
  float* av = vs + kMcL * kMcCols;
  float* Mv = av + kMcL;
  float* bv = Mv + kMcL;
  float* us = bv + kMcL;
  pdl_wait();
  pdl_trigger();
  const int blk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kMcCols;
  const int4 e = reinterpret_cast<const int4*>(a.ent)[p.tiles[2 * blk]];
  const int t0 = p.tiles[2 * blk + 1], len = min(kMcL, e.z - t0);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const float ib = a.i_bias ? a.i_bias[h] : 0.f, fb = a.f_bias ? a.f_bias[h] : 0.f;
  mlstm_load_kv_gates(proj + (size_t)(e.y + t0) * a.ldp, a, h, len, c0, 1.f, ib, fb, (float*)nullptr, kT, vs, av, bv, false);
  __syncthreads();
  mlstm_block_scan(-INFINITY, av, bv, Mv);
  __syncthreads();
  const float A = Mv[kMcL - 1];
  if (tid < kMcL) us[tid] = expf(av[tid] - A);
  __syncthreads();
  float* Ug = p.cS + ((size_t)blk * a.H + h) * D * a.V;
  float* nUg = p.cn + ((size_t)blk * a.H + h) * D;
  for (int dbase = 0; dbase < D; dbase += 128) {
    float acc[8][4] = {};
    float nacc[8] = {};
    for (int sidx = 0; sidx < len; ++sidx) {
      const float u = us[sidx];
      const float4 vb = *reinterpret_cast<const float4*>(vs + sidx * kMcCols + 4 * tx);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int d = dbase + ty + 16 * r;
        const float uk = d < D ? u * kT[d * kMcLp + sidx] : 0.f;
        acc[r][0] = fmaf(uk, vb.x, acc[r][0]); acc[r][1] = fmaf(uk, vb.y, acc[r][1]);
        acc[r][2] = fmaf(uk, vb.z, acc[r][2]); acc[r][3] = fmaf(uk, vb.w, acc[r][3]);
        nacc[r] += uk;
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int d = dbase + ty + 16 * r;
      if (d >= D) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + 4 * tx + j;
        if (c < a.V) Ug[(size_t)d * a.V + c] = acc[r][j];
      }
      if (tx == 0 && blockIdx.z == 0) nUg[d] = nacc[r];
    }
  }
  if (tid == 0 && blockIdx.z == 0) {
    float* sc = p.csc + ((size_t)blk * a.H + h) * 4;
    sc[0] = bv[kMcL - 1];
    sc[1] = A;
  }
}

// pass 2: one thread per state element (the D*V entries of S, then the D entries of n), blocks of the entry in order
__global__ void __launch_bounds__(256)
mlstm_par_carry_kernel(MlstmArgs a, MlstmPar p, int n_tiles) {
  pdl_wait();
  pdl_trigger();
  const int ent_i = blockIdx.x, h = blockIdx.y;
  const int4 e = reinterpret_cast<const int4*>(a.ent)[ent_i];
  const size_t DV = (size_t)a.D * a.V, total = DV + a.D;
  const size_t idx = (size_t)blockIdx.z * blockDim.x + threadIdx.x;
  int first = 0;
  while (first < n_tiles && p.tiles[2 * first] != ent_i) ++first;
  const int nblk = (e.z + kMcL - 1) / kMcL;
  const bool fresh = e.w == 0;
  float* mg = a.m + (size_t)e.x * a.H + h;
  float m0 = fresh ? 0.f : *mg;
  float* state = nullptr;
  if (idx < DV) state = a.S + ((size_t)e.x * a.H + h) * DV + idx;
  else if (idx < total) state = a.n + ((size_t)e.x * a.H + h) * a.D + (idx - DV);
  float sv = (state && !fresh) ? *state : 0.f;
  // eight blocks at a time: all their loads are issued before the first store, so the chain is the arithmetic only
  for (int b0 = 0; b0 < nblk; b0 += 8) {
    float bL[8], A[8], u[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int blk = first + min(b0 + j, nblk - 1);
      const float* sc = p.csc + ((size_t)blk * a.H + h) * 4;
      bL[j] = sc[0];
      A[j] = sc[1];
      u[j] = 0.f;
      if (state) u[j] = idx < DV ? p.cS[((size_t)blk * a.H + h) * DV + idx] : p.cn[((size_t)blk * a.H + h) * a.D + (idx - DV)];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (b0 + j >= nblk) break;
      const int blk = first + b0 + j;
      const float M = fmaxf(m0, A[j]), g = expf(m0 - M), w = expf(A[j] - M);
      if (state) {
        float* slot = idx < DV ? p.cS + ((size_t)blk * a.H + h) * DV + idx : p.cn + ((size_t)blk * a.H + h) * a.D + (idx - DV);
        *slot = sv;
        sv = g * sv + w * u[j];
      }
      if (idx == 0) p.csc[((size_t)blk * a.H + h) * 4 + 2] = m0;
      m0 = bL[j] + M;
    }
  }
  if (state) *state = sv;
  // the slot's m is read by every CTA of this pass: its new value waits in the last block's scalars until pass 3
  if (idx == 0) p.csc[((size_t)(first + nblk - 1) * a.H + h) * 4 + 3] = m0;
}

template <typename E>
__global__ void __launch_bounds__(kMcThreads)
mlstm_par_readout_kernel(const E* __restrict__ proj, float* __restrict__ o, MlstmArgs a, MlstmPar p) {
  extern __shared__ __align__(16) float smc[];
  const int D = a.D;
  float* qT = smc;
  float* kT = qT + (size_t)D * kMcLp;
  float* Ss = kT + (size_t)D * kMcLp;
  float* AT = Ss + (size_t)D * kMcCols;
  float* vs = AT + kMcL * kMcLp;
  float* ns = vs + kMcL * kMcCols;
  float* av = ns + D;
  float* Mv = av + kMcL;
  float* bv = Mv + kMcL;
  float* qn = bv + kMcL;
  pdl_wait();
  pdl_trigger();
  const int blk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kMcCols;
  const int4 e = reinterpret_cast<const int4*>(a.ent)[p.tiles[2 * blk]];
  const int t0 = p.tiles[2 * blk + 1], len = min(kMcL, e.z - t0);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const float ib = a.i_bias ? a.i_bias[h] : 0.f, fb = a.f_bias ? a.f_bias[h] : 0.f;
  const float* Sin = p.cS + ((size_t)blk * a.H + h) * D * a.V;
  const float* nin = p.cn + ((size_t)blk * a.H + h) * D;
  const float m0 = p.csc[((size_t)blk * a.H + h) * 4 + 2];
  if (tid == 0 && blockIdx.z == 0 && t0 + kMcL >= e.z)
    a.m[(size_t)e.x * a.H + h] = p.csc[((size_t)blk * a.H + h) * 4 + 3];
  for (int i = tid; i < D * kMcCols; i += kMcThreads) {
    const int d = i / kMcCols, c = c0 + i % kMcCols;
    Ss[i] = c < a.V ? Sin[(size_t)d * a.V + c] : 0.f;
  }
  for (int d = tid; d < D; d += kMcThreads) ns[d] = nin[d];
  mlstm_load_kv_gates(proj + (size_t)(e.y + t0) * a.ldp, a, h, len, c0, 1.f / sqrtf((float)D), ib, fb, qT, kT, vs, av, bv, true);
  __syncthreads();
  mlstm_block_scan(m0, av, bv, Mv);
  __syncthreads();
  {
    float acc[4][4] = {};
#pragma unroll 4
    for (int d = 0; d < D; ++d) {
      const float4 qa = *reinterpret_cast<const float4*>(qT + d * kMcLp + 4 * ty);
      const float4 kb = *reinterpret_cast<const float4*>(kT + d * kMcLp + 4 * tx);
      const float qv[4] = {qa.x, qa.y, qa.z, qa.w}, kv[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = 4 * ty + i, sidx = 4 * tx + j;
        AT[sidx * kMcLp + t] = (sidx <= t) ? acc[i][j] * expf(av[sidx] - Mv[t]) : 0.f;
      }
  }
  if (tid < kMcL) {
    float d0 = 0.f;
    for (int d = 0; d < D; ++d) d0 = fmaf(ns[d], qT[d * kMcLp + tid], d0);
    qn[tid] = d0;
  }
  __syncthreads();
  float inter[4][4] = {}, intra[4][4] = {};
#pragma unroll 4
  for (int d = 0; d < D; ++d) {
    const float4 qa = *reinterpret_cast<const float4*>(qT + d * kMcLp + 4 * ty);
    const float4 sb = *reinterpret_cast<const float4*>(Ss + d * kMcCols + 4 * tx);
    const float qv[4] = {qa.x, qa.y, qa.z, qa.w}, sv[4] = {sb.x, sb.y, sb.z, sb.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) inter[i][j] = fmaf(qv[i], sv[j], inter[i][j]);
  }
  float rowsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
  for (int sidx = 0; sidx < len; ++sidx) {
    const float4 aa = *reinterpret_cast<const float4*>(AT + sidx * kMcLp + 4 * ty);
    const float4 vb = *reinterpret_cast<const float4*>(vs + sidx * kMcCols + 4 * tx);
    const float aw[4] = {aa.x, aa.y, aa.z, aa.w}, vv[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      rowsum[i] += aw[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) intra[i][j] = fmaf(aw[i], vv[j], intra[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = 4 * ty + i;
    if (t >= len) continue;
    const float g = expf(m0 - Mv[t]);
    const float den = fmaxf(fabsf(g * qn[t] + rowsum[i]), expf(-(bv[t] + Mv[t]))) + 1e-6f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + 4 * tx + j;
      if (c < a.V) o[((size_t)(e.y + t0 + t) * a.H + h) * a.V + c] = (g * inter[i][j] + intra[i][j]) / den;
    }
  }
}

static size_t mlstm_chunk_smem(int D) {
  return sizeof(float) * (2 * (size_t)D * kMcLp + (size_t)D * kMcCols + kMcL * kMcLp + kMcL * kMcCols + D + 5 * kMcL);
}

// y[row, h, :] = o / rms(o over the head) * w[h, :] * sigmoid(gate[row, h, :]); one warp per (row, head).
template <typename E>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o, const E* __restrict__ proj, const float* __restrict__ w, E* __restrict__ y,
                 int rows, int H, int V, int ldp, int g_off, float eps) {
  pdl_wait();
  pdl_trigger();
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= rows * H) return;
  const int row = item / H, h = item % H;
  const float* orow = o + (size_t)item * V;
  float ss = 0.f;
  for (int c = lane; c < V; c += 32) ss += orow[c] * orow[c];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / V + eps);
  for (int c = lane; c < V; c += 32) {
    const float g = 1.f / (1.f + expf(-m_to_f(proj[(size_t)row * ldp + g_off + h * V + c])));
    y[(size_t)item * V + c] = m_from_f<E>(orow[c] * r * w[h * V + c] * g);
  }
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_mlstm_ragged(const void* proj, float* o_scratch, void* y, const int32_t* ent, int n_ent, int rows, int H, int D,
                     int V, int ldp, int q_off, int k_off, int v_off, int i_off, int f_off, int g_off,
                     const float* i_bias, const float* f_bias, float cap, const float* out_w, float eps, float* S,
                     float* n, float* m, int blocked, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(proj && o_scratch && y && ent && out_w && S && n && m, "dli_mlstm_ragged: null pointer");
  DLI_CHECK_ARG(H > 0 && D > 0 && V > 0, "dli_mlstm_ragged: empty shape");
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_mlstm_ragged: ent must be 16-byte aligned");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0 || n_ent <= 0) return DLI_OK;
  MlstmArgs a{ent, H, D, V, ldp, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, S, n, m};
  const size_t smem = sizeof(float) * ((size_t)D * kMlCols + 3 * (size_t)D + kMlThreads + kMlGroups);
  DLI_CHECK_ARG(smem <= 200 * 1024, "dli_mlstm_ragged: key size %d needs %zu bytes of shared memory", D, smem);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(n_ent, H, (V + kMlCols - 1) / kMlCols);
  const size_t csmem = mlstm_chunk_smem(D);
  const bool chunked = blocked && csmem <= 220 * 1024;  // larger key sizes: the token-by-token kernel
  const dim3 cgrid(n_ent, H, (V + kMcCols - 1) / kMcCols);
  if (dt == 0) {
    static PerDeviceOnce once;
    DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                        DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_chunk_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)));
    if (chunked) DLI_LAUNCH("mlstm_chunk", mlstm_chunk_kernel<bf16>, cgrid, dim3(kMcThreads), csmem, s, (const bf16*)proj, o_scratch, a);
    else DLI_LAUNCH("mlstm_scan", mlstm_scan_kernel<bf16>, grid, dim3(kMlThreads), smem, s, (const bf16*)proj, o_scratch, a);
    DLI_LAUNCH("mlstm_out", mlstm_out_kernel<bf16>, dim3((rows * H + 3) / 4), dim3(128), 0, s, (const float*)o_scratch, (const bf16*)proj, out_w, (bf16*)y, rows, H, V, ldp, g_off, eps);
  } else {
    static PerDeviceOnce once;
    DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                        DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_chunk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)));
    if (chunked) DLI_LAUNCH("mlstm_chunk", mlstm_chunk_kernel<float>, cgrid, dim3(kMcThreads), csmem, s, (const float*)proj, o_scratch, a);
    else DLI_LAUNCH("mlstm_scan", mlstm_scan_kernel<float>, grid, dim3(kMlThreads), smem, s, (const float*)proj, o_scratch, a);
    DLI_LAUNCH("mlstm_out", mlstm_out_kernel<float>, dim3((rows * H + 3) / 4), dim3(128), 0, s, (const float*)o_scratch, (const float*)proj, out_w, (float*)y, rows, H, V, ldp, g_off, eps);
  }
  return DLI_OK;
}

size_t dli_mlstm_parallel_scratch_floats(int n_tiles, int H, int D, int V) {
  return (size_t)n_tiles * H * ((size_t)D * V + D + 4);
}

int dli_mlstm_ragged_parallel(const void* proj, float* o_scratch, void* y, const int32_t* ent, int n_ent,
                              const int32_t* tiles, int n_tiles, float* scratch, int rows, int H, int D, int V, int ldp,
                              int q_off, int k_off, int v_off, int i_off, int f_off, int g_off, const float* i_bias,
                              const float* f_bias, float cap, const float* out_w, float eps, float* S, float* n, float* m,
                              int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(proj && o_scratch && y && ent && tiles && scratch && out_w && S && n && m, "dli_mlstm_ragged_parallel: null pointer");
  DLI_CHECK_ARG(H > 0 && D > 0 && V > 0, "dli_mlstm_ragged_parallel: empty shape");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  const size_t csmem = mlstm_chunk_smem(D);
  if (csmem > 220 * 1024) return dli::fail(DLI_ERR_UNSUPPORTED, "dli_mlstm_ragged_parallel: key size %d is too large for the block form", D);
  if (rows <= 0 || n_ent <= 0 || n_tiles <= 0) return DLI_OK;
  MlstmArgs a{ent, H, D, V, ldp, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, S, n, m};
  MlstmPar p{tiles, scratch, scratch + (size_t)n_tiles * H * D * V, scratch + (size_t)n_tiles * H * ((size_t)D * V + D)};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 bgrid(n_tiles, H, (V + kMcCols - 1) / kMcCols);
  const size_t lsmem = sizeof(float) * ((size_t)D * kMcLp + kMcL * kMcCols + 4 * kMcL);
  const size_t total = (size_t)D * V + D;
  const dim3 cgrid(n_ent, H, (unsigned)((total + 255) / 256));
  if (dt == 0) {
    static PerDeviceOnce once;
    DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_par_local_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
                        DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_par_readout_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)));
    DLI_LAUNCH("mlstm_par_local", mlstm_par_local_kernel<bf16>, bgrid, dim3(kMcThreads), lsmem, s, (const bf16*)proj, a, p);
    DLI_LAUNCH("mlstm_par_carry", mlstm_par_carry_kernel, cgrid, dim3(256), 0, s, a, p, n_tiles);
    DLI_LAUNCH("mlstm_par_readout", mlstm_par_readout_kernel<bf16>, bgrid, dim3(kMcThreads), csmem, s, (const bf16*)proj, o_scratch, a, p);
    DLI_LAUNCH("mlstm_out", mlstm_out_kernel<bf16>, dim3((rows * H + 3) / 4), dim3(128), 0, s, (const float*)o_scratch, (const bf16*)proj, out_w, (bf16*)y, rows, H, V, ldp, g_off, eps);
  } else {
    static PerDeviceOnce once;
    DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_par_local_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
                        DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_par_readout_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)));
    DLI_LAUNCH("mlstm_par_local", mlstm_par_local_kernel<float>, bgrid, dim3(kMcThreads), lsmem, s, (const float*)proj, a, p);
    DLI_LAUNCH("mlstm_par_carry", mlstm_par_carry_kernel, cgrid, dim3(256), 0, s, a, p, n_tiles);
    DLI_LAUNCH("mlstm_par_readout", mlstm_par_readout_kernel<float>, bgrid, dim3(kMcThreads), csmem, s, (const float*)proj, o_scratch, a, p);
    DLI_LAUNCH("mlstm_out", mlstm_out_kernel<float>, dim3((rows * H + 3) / 4), dim3(128), 0, s, (const float*)o_scratch, (const float*)proj, out_w, (float*)y, rows, H, V, ldp, g_off, eps);
  }
  return DLI_OK;
}

}  // extern "C"
