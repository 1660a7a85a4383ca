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
                     float* n, float* m, int dt, dli_stream_t stream) {
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
  if (dt == 0) {
    static PerDeviceOnce once;
    DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));
    DLI_LAUNCH("mlstm_scan", mlstm_scan_kernel<bf16>, grid, dim3(kMlThreads), smem, s, (const bf16*)proj, o_scratch, a);
    DLI_LAUNCH("mlstm_out", mlstm_out_kernel<bf16>, dim3((rows * H + 3) / 4), dim3(128), 0, s, (const float*)o_scratch, (const bf16*)proj, out_w, (bf16*)y, rows, H, V, ldp, g_off, eps);
  } else {
    static PerDeviceOnce once;
    DLI_ONCE_PER_DEVICE(once, dev, DLI_CUDA_CALL(cudaFuncSetAttribute(mlstm_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));
    DLI_LAUNCH("mlstm_scan", mlstm_scan_kernel<float>, grid, dim3(kMlThreads), smem, s, (const float*)proj, o_scratch, a);
    DLI_LAUNCH("mlstm_out", mlstm_out_kernel<float>, dim3((rows * H + 3) / 4), dim3(128), 0, s, (const float*)o_scratch, (const float*)proj, out_w, (float*)y, rows, H, V, ldp, g_off, eps);
  }
  return DLI_OK;
}

}  // extern "C"
