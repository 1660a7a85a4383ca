// Selective state-space mixer (Mamba-2 form) for a RAGGED step.  The input projection's row is laid out as
// [z: H*V | x: H*V | B: G*N | C: G*N | dt: H].  Three kernels:
//   dli_conv1d_act_ragged   causal per-channel convolution over time of a block of projection columns (x, B, C),
//                           with bias and SiLU, reading the sequence's last taps-1 inputs from its state slot and
//                           advancing them -> fp32 rows
//   dli_ssm_scan_ragged     per head h (group g = h / (H/G)):  dt_t = softplus(dt_t + dt_bias_h),
//                           S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T   (S: N x V, fp32, per state slot)
//                           y_t = S_t^T C_t + D_h x_t
//   dli_gated_group_rmsnorm y * silu(z), RMS norm in groups, times a weight per channel -> the out-projection's operand
// Everything that enters the recurrence after the convolution is fp32.  An entry whose first position is 0 starts
// from a zero state and a zero convolution history whatever its slot held before.
#include <math.h>

#include "common.cuh"

namespace dli {

template <typename E> __device__ __forceinline__ float m_to_f(E v);
template <> __device__ __forceinline__ float m_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float m_to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E m_from_f(float v);
template <> __device__ __forceinline__ float m_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 m_from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float m_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// out[row, c] = act(bias[c] + sum_j w[c, j] * in[t - taps + 1 + j, c]); in = columns [off, off + C) of proj.
// Inputs before the entry's first row come from tail [slots, taps-1, C] (oldest first), zeros before position 0.
// single != 0 (one row per entry): the channel's thread also shifts the slot's tail, so no second kernel is needed.
template <typename E>
__global__ void __launch_bounds__(256)
conv1d_act_kernel(const E* __restrict__ proj, float* __restrict__ tail, const float* __restrict__ w,
                  const float* __restrict__ bias, const int32_t* __restrict__ row_ent, const int32_t* __restrict__ ent,
                  float* __restrict__ out, int C, int taps, int ldp, int off, int act, int single) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int4 e = reinterpret_cast<const int4*>(ent)[row_ent[row]];  // slot, row0, n, start
  const int back = row - e.y, pos = e.w + back;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += blockDim.x * gridDim.y) {
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int dist = taps - 1 - j;
      if (pos - dist < 0) continue;
      float v;
      if (dist <= back) v = m_to_f(proj[(size_t)(row - dist) * ldp + off + c]);
      else v = tail[((size_t)e.x * (taps - 1) + (taps - 1 - (dist - back))) * C + c];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    if (act == 1) acc = acc / (1.f + expf(-acc));
    out[(size_t)row * C + c] = acc;
    if (single && taps > 1) {  // every old entry was read above; slot i takes old slot i + 1, the last one the current input
      float* t = tail + (size_t)e.x * (taps - 1) * C + c;
      for (int i = 0; i + 1 < taps - 1; ++i) t[(size_t)i * C] = (pos - (taps - 2 - i) >= 0) ? t[(size_t)(i + 1) * C] : 0.f;
      t[(size_t)(taps - 2) * C] = m_to_f(proj[(size_t)row * ldp + off + c]);
    }
  }
}

// After the convolution: the slot's tail becomes the last taps-1 inputs of the sequence.
template <typename E>
__global__ void __launch_bounds__(256)
conv1d_tail_kernel(const E* __restrict__ proj, float* __restrict__ tail, const int32_t* __restrict__ ent, int C, int taps,
                   int ldp, int off) {
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(ent)[blockIdx.x];
  const int keep = taps - 1, end = e.w + e.z;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += blockDim.x * gridDim.y) {
    float* t = tail + (size_t)e.x * keep * C + c;
    for (int i = 0; i < keep; ++i) {  // ascending: slot i reads old slot i + n (n >= 1), never one already written
      const int p = end - keep + i;
      float v = 0.f;
      if (p >= e.w) v = m_to_f(proj[(size_t)(e.y + p - e.w) * ldp + off + c]);
      else if (p >= 0) v = t[(size_t)(keep - (e.w - p)) * C];
      t[(size_t)i * C] = v;
    }
  }
}

struct SsmRun {
  const int32_t* ent;
  int H, V, N, G;
  int ldx;                  // row stride of xbc (fp32 [rows, H*V + 2*G*N]: x | B | C)
  int ldp, dt_off;          // the projection row's stride and the column of dt
  const float* dt_bias;     // [H]
  const float* a_log;       // [H]
  const float* d_skip;      // [H]
  int np;                   // threads that share one value column (a power of two <= 32); each holds N/np state rows
  int vc;                   // value columns per CTA
};

constexpr int kSsmMaxPerThread = 16;

// Grid (entries, heads, ceil(V / vc)); the CTA walks the entry's rows in order with its part of the state in
// registers: thread (v, p) holds S[n, v] for n = p, p + np, ...
template <typename E>
__global__ void __launch_bounds__(256)
ssm_scan_kernel(const float* __restrict__ xbc, const E* __restrict__ proj, float* __restrict__ S, float* __restrict__ y,
                SsmRun a) {
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(a.ent)[blockIdx.x];  // slot, row0, n, start
  const int h = blockIdx.y, g = h / (a.H / a.G);
  const int p = threadIdx.x % a.np, vl = threadIdx.x / a.np;
  const int v = blockIdx.z * a.vc + vl;
  const bool active = vl < a.vc && v < a.V;
  const int inner = a.H * a.V;
  float s[kSsmMaxPerThread];
  float* Sp = S + (((size_t)e.x * a.H + h) * a.N) * a.V;
#pragma unroll
  for (int i = 0; i < kSsmMaxPerThread; ++i) {
    const int n = p + i * a.np;
    s[i] = (active && n < a.N && e.w > 0) ? Sp[(size_t)n * a.V + v] : 0.f;
  }
  const float na = -expf(a.a_log[h]), db = a.dt_bias[h], dk = a.d_skip[h];
  for (int t = 0; t < e.z; ++t) {
    const size_t row = (size_t)e.y + t;
    const float* xr = xbc + row * a.ldx;
    const float draw = m_to_f(proj[row * a.ldp + a.dt_off + h]) + db;
    const float dt = draw > 20.f ? draw : log1pf(expf(draw));
    const float decay = expf(na * dt);
    const float xv = active ? xr[h * a.V + v] : 0.f;
    const float* Bt = xr + inner + g * a.N;
    const float* Ct = xr + inner + a.G * a.N + g * a.N;
    const float bx = dt * xv;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kSsmMaxPerThread; ++i) {
      const int n = p + i * a.np;
      if (n < a.N) {
        s[i] = fmaf(decay, s[i], Bt[n] * bx);
        acc = fmaf(s[i], Ct[n], acc);
      }
    }
    for (int o = a.np >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (active && p == 0) y[row * inner + h * a.V + v] = acc + dk * xv;
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < kSsmMaxPerThread; ++i) {
      const int n = p + i * a.np;
      if (n < a.N) Sp[(size_t)n * a.V + v] = s[i];
    }
  }
}


// ---- the same recurrence 64 rows at a time (steps with portions of prompts) -------------------------------------
// With a_t = -exp(A_log) dt_t and c_t = a_1 + .. + a_t inside a block that starts from state S_in:
//   y_t   = exp(c_t) C_t^T S_in + sum_{s<=t} exp(c_t - c_s) dt_s (C_t . B_s) x_s + D x_t
//   S_out = exp(c_L) S_in + sum_s exp(c_L - c_s) dt_s B_s x_s^T
// Every exponent is <= 0, so nothing needs rescaling.  One CTA per (entry, head) walks the entry's blocks in order
// with the state in shared memory; each block is four small fp32 matrix products on 64 x 64 output tiles, 4 x 4
// outputs per thread (thread (r, c) owns rows r + 16 i and columns c + 16 j: conflict-free shared-memory reads).
constexpr int kSsmL = 64;

static inline size_t ssm_blocked_smem_bytes(int N, int V) {
  return sizeof(float) * ((size_t)2 * kSsmL * (N + 1) + (size_t)kSsmL * V + (size_t)N * V + (size_t)kSsmL * (kSsmL + 1) + 3 * kSsmL);
}

//
// When an entry spans several blocks they run in parallel (mode 1, carry, mode 3): every block first computes what it
// adds to the state as if it started from nothing (U_c = sum_s e^(c_L - c_s) dt_s B_s x_s^T, and its decay e^(c_L)),
// an elementwise pass carries the state over the blocks in order (S <- e^(c_L) S + U_c, leaving each block's
// incoming state where U_c was), then all blocks compute their outputs from their incoming states.
//   mode 0: one CTA per (entry, head) walks the blocks in order;  mode 1 / 3: one CTA per (block, head).
template <typename E, int mode>
__global__ void __launch_bounds__(256)
ssm_scan_blocked_kernel(const float* __restrict__ xbc, const E* __restrict__ proj, float* __restrict__ S,
                        float* __restrict__ y, SsmRun a, const int32_t* __restrict__ tiles,
                        float* __restrict__ scr_u, float* __restrict__ scr_decay) {
  extern __shared__ float sm[];
  const int N = a.N, V = a.V, NP = N + 1, LP = kSsmL + 1;
  float* Bs = sm;                       // [L][N+1]
  float* Cs = Bs + kSsmL * NP;          // [L][N+1]
  float* Xs = Cs + kSsmL * NP;          // [L][V]
  float* St = Xs + kSsmL * V;           // [N][V]
  float* Gs = St + N * V;               // [L][L+1]
  float* cum = Gs + kSsmL * LP;         // [L] running sum of a_t
  float* dts = cum + kSsmL;             // [L]
  float* wl = dts + kSsmL;              // [L] exp(c_L - c_s) dt_s
  pdl_wait();
  pdl_trigger();
  const int ei = mode == 0 ? (int)blockIdx.x : tiles[2 * blockIdx.x];
  const int4 e = reinterpret_cast<const int4*>(a.ent)[ei];  // slot, row0, n, start
  const int h = blockIdx.y, g = h / (a.H / a.G), tid = threadIdx.x;
  const int tr = tid >> 4, tc = tid & 15;
  const int inner = a.H * V;
  float* Sp = S + (((size_t)e.x * a.H + h) * N) * V;
  float* Up = mode == 0 ? nullptr : scr_u + ((size_t)blockIdx.x * a.H + h) * N * V;
  if (mode == 0) for (int i = tid; i < N * V; i += 256) St[i] = e.w > 0 ? Sp[i] : 0.f;
  if (mode == 1) for (int i = tid; i < N * V; i += 256) St[i] = 0.f;
  if (mode == 3) for (int i = tid; i < N * V; i += 256) St[i] = Up[i];
  const float na = -expf(a.a_log[h]), db = a.dt_bias[h], dk = a.d_skip[h];
  const int b_first = mode == 0 ? 0 : tiles[2 * blockIdx.x + 1];
  const int b_end = mode == 0 ? e.z : min(e.z, b_first + kSsmL);
  for (int b0 = b_first; b0 < b_end; b0 += kSsmL) {
    const int nb = min(kSsmL, e.z - b0);
    __syncthreads();  // the previous block's reads of Bs, Cs, Xs, Gs are done; St is complete
    for (int i = tid; i < kSsmL * N; i += 256) {
      const int t = i / N, n = i - t * N;
      const float* xr = xbc + (size_t)(e.y + b0 + t) * a.ldx + inner;
      Bs[t * NP + n] = t < nb ? xr[g * N + n] : 0.f;
      Cs[t * NP + n] = t < nb ? xr[a.G * N + g * N + n] : 0.f;
    }
    for (int i = tid; i < kSsmL * V; i += 256) {
      const int t = i / V, v = i - t * V;
      Xs[i] = t < nb ? xbc[(size_t)(e.y + b0 + t) * a.ldx + h * V + v] : 0.f;
    }
    if (tid < kSsmL) {
      float dt = 0.f;
      if (tid < nb) {
        const float draw = m_to_f(proj[(size_t)(e.y + b0 + tid) * a.ldp + a.dt_off + h]) + db;
        dt = draw > 20.f ? draw : log1pf(expf(draw));
      }
      dts[tid] = dt;
      cum[tid] = na * dt;
    }
    __syncthreads();
    if (tid == 0) {  // 64 additions in order: the same sums whatever the block's length
      float c = 0.f;
      for (int t = 0; t < kSsmL; ++t) { c += cum[t]; cum[t] = c; }
    }
    __syncthreads();
    if (tid < kSsmL) wl[tid] = expf(cum[kSsmL - 1] - cum[tid]) * dts[tid];
    // G[t][s] = (C_t . B_s) exp(c_t - c_s) dt_s for s <= t
    if (mode != 1) {
      float acc[4][4] = {};
      for (int k = 0; k < N; ++k) {
        float cv[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cv[i] = Cs[(tr + 16 * i) * NP + k];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs[(tc + 16 * j) * NP + k];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(cv[i], bv[j], acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int t = tr + 16 * i, s2 = tc + 16 * j;
          Gs[t * LP + s2] = s2 <= t ? acc[i][j] * expf(cum[t] - cum[s2]) * dts[s2] : 0.f;
        }
    }
    __syncthreads();
    // y[t][v] = sum_s G[t][s] x[s][v] + exp(c_t) sum_n C[t][n] S[n][v] + D x[t][v]
    for (int v0 = 0; v0 < V && mode != 1; v0 += 64) {
      float acc[4][4] = {}, acs[4][4] = {};
      int vv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) vv[j] = min(v0 + tc + 16 * j, V - 1);
      for (int k = 0; k < kSsmL; ++k) {
        float gv[4], xv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) gv[i] = Gs[(tr + 16 * i) * LP + k];
#pragma unroll
        for (int j = 0; j < 4; ++j) xv[j] = Xs[k * V + vv[j]];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(gv[i], xv[j], acc[i][j]);
      }
      for (int k = 0; k < N; ++k) {
        float cv[4], sv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cv[i] = Cs[(tr + 16 * i) * NP + k];
#pragma unroll
        for (int j = 0; j < 4; ++j) sv[j] = St[k * V + vv[j]];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acs[i][j] = fmaf(cv[i], sv[j], acs[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = tr + 16 * i;
        if (t >= nb) continue;
        const float ec = expf(cum[t]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int v = v0 + tc + 16 * j;
          if (v < V) y[(size_t)(e.y + b0 + t) * inner + h * V + v] = acc[i][j] + ec * acs[i][j] + dk * Xs[t * V + v];
        }
      }
    }
    __syncthreads();  // every read of the incoming state is done
    if (mode == 3) break;
    // S[n][v] = exp(c_L) S[n][v] + sum_s wl[s] B[s][n] x[s][v]
    const float eL = expf(cum[kSsmL - 1]);
    if (mode == 1 && tid == 0) scr_decay[(size_t)blockIdx.x * a.H + h] = eL;
    for (int n0 = 0; n0 < N; n0 += 64)
      for (int v0 = 0; v0 < V; v0 += 64) {
        float acc[4][4] = {};
        int nn[4], vv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) nn[i] = min(n0 + tr + 16 * i, N - 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) vv[j] = min(v0 + tc + 16 * j, V - 1);
        for (int k = 0; k < kSsmL; ++k) {
          const float w = wl[k];
          float bv[4], xv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) bv[i] = Bs[k * NP + nn[i]] * w;
#pragma unroll
          for (int j = 0; j < 4; ++j) xv[j] = Xs[k * V + vv[j]];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(bv[i], xv[j], acc[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = n0 + tr + 16 * i, v = v0 + tc + 16 * j;
            if (n < N && v < V) St[n * V + v] = eL * St[n * V + v] + acc[i][j];
          }
      }
  }
  __syncthreads();
  if (mode == 0) for (int i = tid; i < N * V; i += 256) Sp[i] = St[i];
  if (mode == 1) for (int i = tid; i < N * V; i += 256) Up[i] = St[i];
}

// The carry over an entry's blocks in order, elementwise: grid (entries, heads, ceil(N*V / 256)).
__global__ void __launch_bounds__(256)
ssm_par_carry_kernel(const int32_t* __restrict__ ent, const int32_t* __restrict__ tiles, int n_tiles, float* __restrict__ S,
                     float* __restrict__ scr_u, const float* __restrict__ scr_decay, int H, int NV) {
  __shared__ int t_first;
  pdl_wait();
  pdl_trigger();
  const int4 e = reinterpret_cast<const int4*>(ent)[blockIdx.x];
  const int h = blockIdx.y;
  if (threadIdx.x == 0) {
    int t = 0;
    while (t < n_tiles && tiles[2 * t] != (int)blockIdx.x) ++t;
    t_first = t;
  }
  __syncthreads();
  const int i = blockIdx.z * 256 + threadIdx.x;
  if (i >= NV) return;
  const int nt = (e.z + kSsmL - 1) / kSsmL;
  float* Sp = S + ((size_t)e.x * H + h) * NV + i;
  float s = e.w > 0 ? *Sp : 0.f;
  for (int c0 = 0; c0 < nt; c0 += 4) {  // four blocks' contributions requested before the first is used
    float u[4], dcy[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const size_t t = (size_t)t_first + min(c0 + k, nt - 1);
      u[k] = scr_u[(t * H + h) * NV + i];
      dcy[k] = scr_decay[t * H + h];
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (c0 + k >= nt) break;
      scr_u[(((size_t)t_first + c0 + k) * H + h) * NV + i] = s;
      s = fmaf(dcy[k], s, u[k]);
    }
  }
  *Sp = s;
}

// out[row] = groupnorm(y[row] * silu(z[row])) * w; z = columns [z_off, z_off + d) of proj.
template <typename E>
__global__ void __launch_bounds__(1024)
gated_group_rmsnorm_kernel(const float* __restrict__ y, const E* __restrict__ proj, const float* __restrict__ w,
                           E* __restrict__ out, int d, int groups, float eps, int ldp, int z_off) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  const int gd = d / groups;
  for (int g = 0; g < groups; ++g) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < gd; c += blockDim.x) {
      const float z = m_to_f(proj[row * ldp + z_off + g * gd + c]);
      const float v = y[row * d + g * gd + c] * (z / (1.f + expf(-z)));
      ss += v * v;
    }
    ss = m_block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / gd + eps);
    for (int c = threadIdx.x; c < gd; c += blockDim.x) {
      const float z = m_to_f(proj[row * ldp + z_off + g * gd + c]);
      const float v = y[row * d + g * gd + c] * (z / (1.f + expf(-z)));
      out[row * d + g * gd + c] = m_from_f<E>(v * r * w[g * gd + c]);
    }
  }
}

}  // namespace dli

using namespace dli;

extern "C" {

int dli_conv1d_act_ragged(const void* proj, float* tail, const float* w, const float* bias, const int32_t* row_ent,
                          const int32_t* ent, float* out, int rows, int n_ent, int C, int taps, int ldp, int off, int act,
                          int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(proj && w && row_ent && ent && out && C > 0 && taps >= 1 && ldp >= off + C && off >= 0,
                "dli_conv1d_act_ragged: null pointer or bad shape");
  DLI_CHECK_ARG(tail || taps == 1, "dli_conv1d_act_ragged: taps > 1 needs a tail state");
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_conv1d_act_ragged: ent must be 16-byte aligned");
  DLI_CHECK_ARG(act == 0 || act == 1, "dli_conv1d_act_ragged: activation %d (0 = none, 1 = silu)", act);
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // few rows (decode): the channels of a row are dealt to several CTAs
  const int gy = rows <= 64 ? (C + 255) / 256 : 1, gyt = n_ent <= 64 ? (C + 255) / 256 : 1;
  const int single = rows == n_ent ? 1 : 0;
  if (dt == 0) DLI_LAUNCH("conv1d_act", conv1d_act_kernel<bf16>, dim3(rows, gy), dim3(256), 0, s, (const bf16*)proj, tail, w, bias, row_ent, ent, out, C, taps, ldp, off, act, single);
  else DLI_LAUNCH("conv1d_act", conv1d_act_kernel<float>, dim3(rows, gy), dim3(256), 0, s, (const float*)proj, tail, w, bias, row_ent, ent, out, C, taps, ldp, off, act, single);
  if (taps > 1 && !single) {
    if (dt == 0) DLI_LAUNCH("conv1d_tail", conv1d_tail_kernel<bf16>, dim3(n_ent, gyt), dim3(256), 0, s, (const bf16*)proj, tail, ent, C, taps, ldp, off);
    else DLI_LAUNCH("conv1d_tail", conv1d_tail_kernel<float>, dim3(n_ent, gyt), dim3(256), 0, s, (const float*)proj, tail, ent, C, taps, ldp, off);
  }
  return DLI_OK;
}

int dli_ssm_scan_ragged(const float* xbc, const void* proj, float* S, float* y, const int32_t* ent, int n_ent, int H, int V,
                        int N, int G, int ldp, int dt_off, const float* dt_bias, const float* a_log, const float* d_skip,
                        int blocked, const int32_t* tiles, int n_tiles, float* scratch, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(xbc && proj && S && y && ent && dt_bias && a_log && d_skip, "dli_ssm_scan_ragged: null pointer");
  DLI_CHECK_ARG(H > 0 && V > 0 && N > 0 && G > 0 && H % G == 0 && N <= 32 * kSsmMaxPerThread,
                "dli_ssm_scan_ragged: H=%d V=%d N=%d G=%d (H %% G == 0, N <= %d)", H, V, N, G, 32 * kSsmMaxPerThread);
  DLI_CHECK_ARG((reinterpret_cast<uintptr_t>(ent) & 15u) == 0, "dli_ssm_scan_ragged: ent must be 16-byte aligned");
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (n_ent <= 0) return DLI_OK;
  const size_t bsmem = ssm_blocked_smem_bytes(N, V);
  if (blocked && bsmem <= 200 * 1024) {
    SsmRun b{ent, H, V, N, G, H * V + 2 * G * N, ldp, dt_off, dt_bias, a_log, d_skip, 0, 0};
    cudaStream_t bs = static_cast<cudaStream_t>(stream);
    // some entry spans several blocks and the caller gave scratch: all blocks in parallel (local, carry, outputs)
    const bool par = tiles && scratch && n_tiles > n_ent;
    float* scr_u = scratch;
    float* scr_d = par ? scratch + (size_t)n_tiles * H * N * V : nullptr;
#define SSM_BLOCKED_LAUNCH(T, MODE, GRID, WHAT)                                                                              \
  do {                                                                                                                      \
    static PerDeviceOnce once;                                                                                              \
    DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(ssm_scan_blocked_kernel<T, MODE>,                     \
                                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024))); \
    DLI_LAUNCH(WHAT, (ssm_scan_blocked_kernel<T, MODE>), GRID, dim3(256), bsmem, bs, xbc, (const T*)proj, S, y, b, tiles, scr_u, \
               scr_d);                                                                                                      \
  } while (0)
    if (!par) {
      if (dt == 0) SSM_BLOCKED_LAUNCH(bf16, 0, dim3(n_ent, H), "ssm_scan_blocked");
      else SSM_BLOCKED_LAUNCH(float, 0, dim3(n_ent, H), "ssm_scan_blocked");
      return DLI_OK;
    }
    if (dt == 0) SSM_BLOCKED_LAUNCH(bf16, 1, dim3(n_tiles, H), "ssm_par_local");
    else SSM_BLOCKED_LAUNCH(float, 1, dim3(n_tiles, H), "ssm_par_local");
    DLI_LAUNCH("ssm_par_carry", ssm_par_carry_kernel, dim3(n_ent, H, (N * V + 255) / 256), dim3(256), 0, bs, ent, tiles, n_tiles,
               S, scr_u, (const float*)scr_d, H, N * V);
    if (dt == 0) SSM_BLOCKED_LAUNCH(bf16, 3, dim3(n_tiles, H), "ssm_par_out");
    else SSM_BLOCKED_LAUNCH(float, 3, dim3(n_tiles, H), "ssm_par_out");
#undef SSM_BLOCKED_LAUNCH
    return DLI_OK;
  }
  int np = 1;
  while (np * kSsmMaxPerThread < N) np <<= 1;
  // few value columns per CTA: a scan is one dependent chain per entry and head, so the columns are what spreads it
  // over the SMs
  int vc = 256 / np;
  while (vc > 8 && (long)n_ent * H * ((V + vc - 1) / vc) < 2L * sm_count_cached()) vc >>= 1;
  if (vc > V) vc = V;
  const int threads = ((vc * np + 31) / 32) * 32;
  SsmRun a{ent, H, V, N, G, H * V + 2 * G * N, ldp, dt_off, dt_bias, a_log, d_skip, np, vc};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(n_ent, H, (V + vc - 1) / vc);
  if (dt == 0) DLI_LAUNCH("ssm_scan", ssm_scan_kernel<bf16>, grid, dim3(threads), 0, s, xbc, (const bf16*)proj, S, y, a);
  else DLI_LAUNCH("ssm_scan", ssm_scan_kernel<float>, grid, dim3(threads), 0, s, xbc, (const float*)proj, S, y, a);
  return DLI_OK;
}

size_t dli_ssm_parallel_scratch_floats(int n_tiles, int H, int N, int V) {
  return (size_t)n_tiles * H * ((size_t)N * V + 1);
}

int dli_gated_group_rmsnorm(const float* y, const void* proj, const float* w, void* out, int rows, int d, int groups,
                            float eps, int ldp, int z_off, int dt, dli_stream_t stream) {
  DLI_CHECK_ARG(y && proj && w && out && d > 0 && groups > 0 && d % groups == 0 && ldp >= z_off + d && z_off >= 0,
                "dli_gated_group_rmsnorm: null pointer, or size %d is not a multiple of %d groups", d, groups);
  DLI_CHECK_ARG(dt == 0 || dt == 1, "element type %d: 0 = bf16, 1 = float", dt);
  if (rows <= 0) return DLI_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int th = (rows <= 64 && d / groups >= 2048) ? 1024 : 256;  // few rows of a wide model: more threads per row
  if (dt == 0) DLI_LAUNCH("gated_group_rmsnorm", gated_group_rmsnorm_kernel<bf16>, dim3(rows), dim3(th), 0, s, y, (const bf16*)proj, w, (bf16*)out, d, groups, eps, ldp, z_off);
  else DLI_LAUNCH("gated_group_rmsnorm", gated_group_rmsnorm_kernel<float>, dim3(rows), dim3(th), 0, s, y, (const float*)proj, w, (float*)out, d, groups, eps, ldp, z_off);
  return DLI_OK;
}

}  // extern "C"
