// Linear attention with a constant decay per head: per head a d x dv memory S, from the state the request's slot holds,
//   S_t = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t
// with q, k (heads x d) and v (heads x dv) column ranges of one 32-bit projection, each passed through an activation on
// the way in (0: none, 1: silu). The memory, the products and the sums are 32-bit in both run dtypes; o is written in
// 32-bit for the norm that follows.
//
// A block serves 128 / L columns of one head of one request; a column's d numbers are dealt out over L lanes (row i on
// lane i % L), NS = ceil(d / L) per lane in registers. Tokens are staged sixteen at a time in shared memory (q and k of
// the head, v of the block's columns) and walked strictly in order, so a sequence may be cut anywhere without a
// memory seeing other operations or another order.
#include "common.cuh"

namespace tmk {

constexpr int kDecayThreads = 128;
constexpr int kDecayTokens = 16;

__device__ __forceinline__ float act_in(float v, int act) { return act == 1 ? v / (1.0f + expf(-v)) : v; }

template <int NS, int L>
__global__ void __launch_bounds__(kDecayThreads) decay_memory_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int act, const float* __restrict__ decay,
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ y, int heads, int d, int dv) {
  constexpr int CB = kDecayThreads / L;
  extern __shared__ __align__(16) float smem[];
  float* s_q = smem;                                // [16][d]
  float* s_k = s_q + kDecayTokens * d;              // [16][d]
  float* s_v = s_k + kDecayTokens * d;              // [16][CB]

  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.z, h = blockIdx.y;
  const int q0 = cu_q[s], q_len = cu_q[s + 1] - q0;
  if (q_len <= 0) return;
  const int c0 = blockIdx.x * CB;
  const int lane = threadIdx.x % L, cl = threadIdx.x / L;
  const int col = c0 + cl;
  const bool live = col < dv;
  // a request's memories: [heads][d][dv]
  float* S_col = state + (size_t)state_slots[s] * state_stride + state_off + (size_t)h * d * dv + (live ? col : 0);
  const float a = decay[h];

  float S[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int i = lane + L * j;
    S[j] = (live && i < d) ? S_col[(size_t)i * dv] : 0.f;
  }

  for (int t0 = 0; t0 < q_len; t0 += kDecayTokens) {
    const int nt = min(kDecayTokens, q_len - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * d; i += kDecayThreads) {
      const int tt = i / d, e = i - tt * d;
      const float* row = proj + (size_t)(q0 + t0 + tt) * ld;
      s_q[i] = act_in(row[q_col + h * d + e], act);
      s_k[i] = act_in(row[k_col + h * d + e], act);
    }
    for (int i = threadIdx.x; i < nt * CB; i += kDecayThreads) {
      const int tt = i / CB, cc = i - tt * CB;
      s_v[i] = c0 + cc < dv ? act_in(proj[(size_t)(q0 + t0 + tt) * ld + v_col + h * dv + c0 + cc], act) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float v = s_v[tt * CB + cl];
      const float* qv = s_q + tt * d;
      const float* kv = s_k + tt * d;
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        const int i = lane + L * j;
        if (i < d) {
          S[j] = fmaf(a, S[j], kv[i] * v);
          o = fmaf(S[j], qv[i], o);
        }
      }
#pragma unroll
      for (int off = L / 2; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (lane == 0 && live) y[(size_t)(q0 + t0 + tt) * heads * dv + (size_t)h * dv + col] = o;
    }
  }
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int i = lane + L * j;
    if (live && i < d) S_col[(size_t)i * dv] = S[j];
  }
}

template <int NS, int L>
int launch_decay_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int act, const float* decay, float* state,
                        long long state_stride, long long state_off, const int* cu_q, const int* state_slots, float* y,
                        int n_seqs, int heads, int d, int dv, cudaStream_t stream) {
  constexpr int CB = kDecayThreads / L;
  const size_t smem = sizeof(float) * kDecayTokens * (2 * (size_t)d + CB);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decay_memory_kernel<NS, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_pdl(decay_memory_kernel<NS, L>, dim3((dv + CB - 1) / CB, heads, n_seqs), dim3(kDecayThreads), smem, stream, proj,
                    ld, q_col, k_col, v_col, act, decay, state, state_stride, state_off, cu_q, state_slots, y, heads, d, dv);
}

}  // namespace tmk

// proj: float, token t's row at proj + t * ld, q at q_col (heads x d), k at k_col, v at v_col (heads x dv); decay [heads]
// float; a request's memories [heads, d, dv] start state_off floats into its slot of `state`; y [T, heads * dv] float.
extern "C" int tm_decay_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int act, const float* decay,
                               float* state, long long state_stride, long long state_off, const int* cu_q, const int* state_slots,
                               float* y, int n_seqs, int heads, int d, int dv, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || d < 1 || dv < 1 || (act != 0 && act != 1)) return TM_ERR_UNSUPPORTED_SHAPE;
#define TM_DECAY(NS_, L_)                                                                                                  \
  return tmk::launch_decay_memory<NS_, L_>(proj, ld, q_col, k_col, v_col, act, decay, state, state_stride, state_off, cu_q, \
                                           state_slots, y, n_seqs, heads, d, dv, stream)
  if (d <= 8) TM_DECAY(2, 4);
  if (d <= 16) TM_DECAY(4, 4);
  if (d <= 32) TM_DECAY(8, 4);
  if (d <= 64) TM_DECAY(16, 4);
  if (d <= 128) TM_DECAY(16, 8);
  if (d <= 256) TM_DECAY(16, 16);
  if (d <= 512) TM_DECAY(32, 16);
#undef TM_DECAY
  return TM_ERR_UNSUPPORTED_SHAPE;
}
