// Linear attention with a constant decay per head: per head a d x dv memory S, from the state the request's slot holds,
//   S_t = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t
// with q, k (heads x d) and v (heads x dv) column ranges of one 32-bit projection, each passed through an activation on
// the way in (0: none, 1: silu). The memory, the products and the sums are 32-bit in both run dtypes; o is written in
// 32-bit for the norm that follows.
//
// A block serves CB = 128 / L columns of one head of one request; a column's d numbers are dealt out over L lanes, NS =
// ceil(d / L) neighbouring rows per lane in registers (row i on lane i / NS), so that a lane reads its part of q and k
// with 16-byte loads. Tokens are staged sixteen at a time in shared memory (q and k of the head, padded with zeros to
// NS * L, v of the block's columns) and walked strictly in order; a token's results wait in shared memory and leave
// together after the walk.
//
// Three ways to run (mode):
//   0  one walk over each request's tokens, from the slot's memory and back into it. A sequence may be cut anywhere
//      into such steps without a memory seeing other operations or another order.
//   1  long portions, first pass: a block walks ONE time slice of slice_len tokens from a zero memory (no q, no
//      results) and leaves the slice's own memory in scratch. tm_decay_pass_states then turns the scratch into every
//      slice's memory at its start (S <- decay^len S + own) and the slot's memory into the one after the last slice.
//   2  third pass: every slice again, from its start memory, now with the results.
#include "common.cuh"

namespace tmk {

constexpr int kDecayThreads = 128;
constexpr int kDecayTokens = 16;

__device__ __forceinline__ float act_in(float v, int act) { return act == 1 ? v / (1.0f + expf(-v)) : v; }

template <int NS> __device__ __forceinline__ void load_rows(const float* p, float (&v)[NS]) {
  if constexpr (NS % 4 == 0) {
#pragma unroll
    for (int j = 0; j < NS; j += 4) {
      const float4 f = *reinterpret_cast<const float4*>(p + j);
      v[j] = f.x, v[j + 1] = f.y, v[j + 2] = f.z, v[j + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < NS; j += 2) {
      const float2 f = *reinterpret_cast<const float2*>(p + j);
      v[j] = f.x, v[j + 1] = f.y;
    }
  }
}

template <int NS, int L, int MODE>
__global__ void __launch_bounds__(kDecayThreads) decay_memory_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int act, const float* __restrict__ decay,
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ y, int heads, int d, int dv, int slice_len, int max_slices,
    float* __restrict__ slice_S) {
  constexpr int CB = kDecayThreads / L;
  constexpr int DP = NS * L;                        // rows, padded
  extern __shared__ __align__(16) float smem[];
  float* s_q = smem;                                // [16][DP]
  float* s_k = s_q + kDecayTokens * DP;             // [16][DP]
  float* s_v = s_k + kDecayTokens * DP;             // [16][CB]
  float* s_o = s_v + kDecayTokens * CB;             // [16][CB]

  pdl_launch_dependents();
  pdl_wait();
  const int s = MODE == 0 ? blockIdx.z : blockIdx.z / max_slices;
  const int k = MODE == 0 ? 0 : blockIdx.z - s * max_slices;
  const int h = blockIdx.y;
  const int q_len = cu_q[s + 1] - cu_q[s];
  const int t_begin = MODE == 0 ? 0 : k * slice_len;
  const int t_end = MODE == 0 ? q_len : min(q_len, t_begin + slice_len);
  if (t_begin >= t_end) return;
  const int q0 = cu_q[s];
  const int c0 = blockIdx.x * CB;
  const int lane = threadIdx.x % L, cl = threadIdx.x / L;
  const int col = c0 + cl;
  const bool live = col < dv;
  // a request's memories: [heads][d][dv]
  float* S_col = (MODE == 0 ? state + (size_t)state_slots[s] * state_stride + state_off
                            : slice_S + (size_t)blockIdx.z * heads * d * dv) + (size_t)h * d * dv + (live ? col : 0);
  const float a = decay[h];

  float S[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int i = lane * NS + j;
    S[j] = (live && i < d && MODE != 1) ? S_col[(size_t)i * dv] : 0.f;
  }

  for (int t0 = t_begin; t0 < t_end; t0 += kDecayTokens) {
    const int nt = min(kDecayTokens, t_end - t0);
    __syncthreads();
    for (int tt = threadIdx.x / 32; tt < nt; tt += kDecayThreads / 32) {
      const float* row = proj + (size_t)(q0 + t0 + tt) * ld;
      for (int e = threadIdx.x % 32; e < DP; e += 32) {
        if (MODE != 1) s_q[tt * DP + e] = e < d ? act_in(row[q_col + h * d + e], act) : 0.f;
        s_k[tt * DP + e] = e < d ? act_in(row[k_col + h * d + e], act) : 0.f;
      }
      for (int cc = threadIdx.x % 32; cc < CB; cc += 32)
        s_v[tt * CB + cc] = c0 + cc < dv ? act_in(row[v_col + h * dv + c0 + cc], act) : 0.f;
    }
    __syncthreads();
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      const float v = s_v[tt * CB + cl];
      float kv[NS], qv[NS];
      load_rows<NS>(s_k + tt * DP + lane * NS, kv);
      if (MODE != 1) load_rows<NS>(s_q + tt * DP + lane * NS, qv);
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        S[j] = fmaf(a, S[j], kv[j] * v);
        if (MODE != 1) o = fmaf(S[j], qv[j], o);
      }
      if (MODE != 1) {
#pragma unroll
        for (int off = L / 2; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
        if (lane == 0) s_o[tt * CB + cl] = o;
      }
    }
    if (MODE != 1) {
      __syncthreads();
      for (int i = threadIdx.x; i < nt * CB; i += kDecayThreads) {
        const int tt = i / CB, cc = i - tt * CB;
        if (c0 + cc < dv) y[(size_t)(q0 + t0 + tt) * heads * dv + (size_t)h * dv + c0 + cc] = s_o[i];
      }
    }
  }
  if (MODE != 2) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int i = lane * NS + j;
      if (live && i < d) S_col[(size_t)i * dv] = S[j];
    }
  }
}

// One thread per (request, head, row, column): slice k's scratch memory becomes the memory at its start, and the slot's
// memory the one after the last slice. decay^len is a 64-bit power rounded once.
__global__ void __launch_bounds__(256) decay_pass_states_kernel(float* __restrict__ state, long long state_stride,
                                                                long long state_off, const int* __restrict__ cu_q,
                                                                const int* __restrict__ state_slots,
                                                                const float* __restrict__ decay, float* __restrict__ slice_S,
                                                                int heads, int d, int dv, int slice_len, int max_slices) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int q_len = cu_q[s + 1] - cu_q[s];
  const long long per = (long long)heads * d * dv;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per || q_len <= 0) return;
  const double a = (double)decay[e / ((long long)d * dv)];
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off + e;
  float S = *slot;
  const int slices = (q_len + slice_len - 1) / slice_len;
  const float a_full = (float)pow(a, (double)slice_len);
  for (int k = 0; k < slices; ++k) {
    const int len = min(slice_len, q_len - k * slice_len);
    const float f = len == slice_len ? a_full : (float)pow(a, (double)len);
    float* mine = slice_S + ((size_t)s * max_slices + k) * per + e;
    const float own = *mine;
    *mine = S;
    S = fmaf(f, S, own);
  }
  *slot = S;
}

template <int NS, int L>
int launch_decay_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int act, const float* decay, float* state,
                        long long state_stride, long long state_off, const int* cu_q, const int* state_slots, float* y,
                        int n_seqs, int heads, int d, int dv, int mode, int slice_len, int max_slices, float* slice_S,
                        cudaStream_t stream) {
  constexpr int CB = kDecayThreads / L;
  const size_t smem = sizeof(float) * kDecayTokens * (2 * (size_t)NS * L + 2 * CB);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
#define TM_DECAY_MODE(M_)                                                                                                   \
  {                                                                                                                         \
    if (smem > 40 * 1024) {                                                                                                 \
      cudaError_t e = cudaFuncSetAttribute(decay_memory_kernel<NS, L, M_>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                           (int)smem);                                                                      \
      if (e != cudaSuccess) return (int)e;                                                                                  \
    }                                                                                                                       \
    return launch_pdl(decay_memory_kernel<NS, L, M_>, dim3((dv + CB - 1) / CB, heads, n_seqs * (M_ == 0 ? 1 : max_slices)), \
                      dim3(kDecayThreads), smem, stream, proj, ld, q_col, k_col, v_col, act, decay, state, state_stride,    \
                      state_off, cu_q, state_slots, y, heads, d, dv, slice_len, max_slices, slice_S);                       \
  }
  if (mode == 0) TM_DECAY_MODE(0)
  if (mode == 1) TM_DECAY_MODE(1)
  TM_DECAY_MODE(2)
#undef TM_DECAY_MODE
}

}  // namespace tmk

// proj: float, token t's row at proj + t * ld, q at q_col (heads x d), k at k_col, v at v_col (heads x dv); decay [heads]
// float; a request's memories [heads, d, dv] start state_off floats into its slot of `state`; y [T, heads * dv] float.
// mode 0: one walk per request. modes 1 and 2: the first and third pass over time slices of slice_len tokens, max_slices
// per request, through slice_S [n_seqs * max_slices, heads, d, dv] (float), with tm_decay_pass_states between.
extern "C" int tm_decay_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int act, const float* decay,
                               float* state, long long state_stride, long long state_off, const int* cu_q, const int* state_slots,
                               float* y, int n_seqs, int heads, int d, int dv, int mode, int slice_len, int max_slices,
                               float* slice_S, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || d < 1 || dv < 1 || (act != 0 && act != 1) || mode < 0 || mode > 2) return TM_ERR_UNSUPPORTED_SHAPE;
  if (mode != 0 && (slice_len < 1 || max_slices < 1 || !slice_S)) return TM_ERR_SCRATCH_TOO_SMALL;
#define TM_DECAY(NS_, L_)                                                                                                  \
  return tmk::launch_decay_memory<NS_, L_>(proj, ld, q_col, k_col, v_col, act, decay, state, state_stride, state_off, cu_q, \
                                           state_slots, y, n_seqs, heads, d, dv, mode, slice_len, max_slices, slice_S, stream)
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

// Between the two passes over time slices (see the top of the file).
extern "C" int tm_decay_pass_states(float* state, long long state_stride, long long state_off, const int* cu_q,
                                    const int* state_slots, const float* decay, float* slice_S, int n_seqs, int heads, int d,
                                    int dv, int slice_len, int max_slices, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || d < 1 || dv < 1 || slice_len < 1 || max_slices < 1 || !slice_S) return TM_ERR_UNSUPPORTED_SHAPE;
  const long long per = (long long)heads * d * dv;
  return tmk::launch_pdl(tmk::decay_pass_states_kernel, dim3((unsigned)((per + 255) / 256), n_seqs), dim3(256), 0, stream, state,
                         state_stride, state_off, cu_q, state_slots, decay, slice_S, heads, d, dv, slice_len, max_slices);
}
