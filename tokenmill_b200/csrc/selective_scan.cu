// Selective scan with one step size per channel and one decay per (channel, state) pair (the first Mamba form).
//
// Per request and channel c, with N states, walking the step's tokens in order from the state the request's slot holds:
//   dt = softplus(W_dt[c, :] . low + b_dt[c])          low: the token's first R numbers of the projection [low | B | C]
//   S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x_c B_n     A = -exp(A_log)
//   y_c = sum_n S[c, n] C_n + D_c x_c                   out_c = y_c silu(z_c)
// x is the convolved and activated input (activation dtype), z the gate's pre-activation (a column range of another
// matrix), [low | B | C] a 32-bit projection. The step size, the exponentials, the state and the sums are 32-bit in
// both run dtypes; W_dt is read in 32-bit, so the rank-R product is part of this kernel.
//
// A block serves 128 / L channels of one request; a channel's N states are dealt out over L lanes (state n on lane
// n % L), NS = ceil(N / L) per lane in registers. Tokens are staged sixteen at a time in shared memory: the projection
// rows, x, z, and the step sizes, which all threads compute together before the walk. Whatever the cut of a sequence
// into steps, a state sees the same operations in the same order.
#include "common.cuh"

namespace tmk {

constexpr int kScanThreads = 128;
constexpr int kScanTokens = 16;

// exp(x) to about one unit in the last place (1.05 at worst, a quarter on average): n = round(x / ln 2), r = x - n ln 2 with ln 2 in two pieces (the
// high one has enough trailing zero bits for n * high to be exact), a degree-7 polynomial on |r| <= 0.347 (remainder below
// 6e-9), then the exponent. Below -86 the result is 0. A decay is multiplied into a state once per token, so its error adds up
// over a sequence: the 32-bit run, whose logits are compared to a few units of 32-bit rounding, takes this form; the
// bfloat16 run takes expf (two units in the last place, on the special-function unit).
__device__ __forceinline__ float exp_one_ulp(float x) {
  if (x < -86.f) return 0.f;
  x = fminf(x, 88.f);
  const float n = rintf(x * 1.4426950408889634f);
  float r = fmaf(n, -0.693145751953125f, x);
  r = fmaf(n, -1.42860682030941723212e-6f, r);
  float p = 1.f / 5040.f;
  p = fmaf(p, r, 1.f / 720.f);
  p = fmaf(p, r, 1.f / 120.f);
  p = fmaf(p, r, 1.f / 24.f);
  p = fmaf(p, r, 1.f / 6.f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p * r, r, r);                 // r + r^2 (1/2 + ...): the small part first, 1 last
  p += 1.f;
  return __int_as_float(__float_as_int(p) + (static_cast<int>(n) << 23));
}

template <typename T> __device__ __forceinline__ float exp_for(float x) { return expf(x); }
template <> __device__ __forceinline__ float exp_for<float>(float x) { return exp_one_ulp(x); }

template <typename T> __device__ __forceinline__ float softplus32(float v) { return v > 20.f ? v : log1pf(exp_for<T>(v)); }

template <typename T, int NS, int L>
__global__ void __launch_bounds__(kScanThreads) selective_scan_kernel(
    const T* __restrict__ x, int inner, const T* __restrict__ zmat, long long z_stride, int z_col,
    const float* __restrict__ dbc, long long dbc_stride, int R, int N, const float* __restrict__ w_dt,
    const float* __restrict__ b_dt, const float* __restrict__ A_log, const float* __restrict__ Dv, float* __restrict__ state,
    long long state_stride, long long state_off, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
    T* __restrict__ out) {
  constexpr int CB = kScanThreads / L;              // channels of a block
  extern __shared__ __align__(16) float smem[];
  const int P = R + 2 * N;
  float* s_dbc = smem;                              // [16][P]
  float* s_x = s_dbc + kScanTokens * P;             // [16][CB]
  float* s_z = s_x + kScanTokens * CB;              // [16][CB]
  float* s_dt = s_z + kScanTokens * CB;             // [16][CB]

  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int q0 = cu_q[s], q_len = cu_q[s + 1] - q0;
  if (q_len <= 0) return;
  const int c0 = blockIdx.x * CB;
  const int lane = threadIdx.x % L, cl = threadIdx.x / L;
  const int c = c0 + cl;
  const bool live = c < inner;
  float* S_row = state + (size_t)state_slots[s] * state_stride + state_off + (size_t)(live ? c : 0) * N;

  float A[NS], S[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = lane + L * j;
    const bool ok = live && n < N;
    A[j] = ok ? -exp_for<T>(A_log[(size_t)c * N + n]) : 0.f;
    S[j] = ok ? S_row[n] : 0.f;
  }
  const float Dc = live ? Dv[c] : 0.f;

  for (int t0 = 0; t0 < q_len; t0 += kScanTokens) {
    const int nt = min(kScanTokens, q_len - t0);
    __syncthreads();                                // the previous tokens' walk has finished with the staging
    for (int i = threadIdx.x; i < nt * P; i += kScanThreads) {
      const int tt = i / P, col = i - tt * P;
      s_dbc[i] = dbc[(size_t)(q0 + t0 + tt) * dbc_stride + col];
    }
    for (int i = threadIdx.x; i < nt * CB; i += kScanThreads) {
      const int tt = i / CB, cc = i - tt * CB;
      const bool ok = c0 + cc < inner;
      s_x[i] = ok ? to_float(x[(size_t)(q0 + t0 + tt) * inner + c0 + cc]) : 0.f;
      s_z[i] = ok ? to_float(zmat[(size_t)(q0 + t0 + tt) * z_stride + z_col + c0 + cc]) : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * CB; i += kScanThreads) {
      const int tt = i / CB, cc = i - tt * CB;
      float dt = 0.f;
      if (c0 + cc < inner) {
        const float* wr = w_dt + (size_t)(c0 + cc) * R;
        const float* low = s_dbc + tt * P;
        float acc = 0.f;
        for (int r = 0; r < R; ++r) acc = fmaf(wr[r], low[r], acc);
        dt = softplus32<T>(acc + b_dt[c0 + cc]);
      }
      s_dt[i] = dt;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = s_dt[tt * CB + cl], xv = s_x[tt * CB + cl];
      const float dx = dt * xv;
      const float* Bv = s_dbc + tt * P + R;
      const float* Cv = Bv + N;
      float y = 0.f;
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        const int n = lane + L * j;
        if (n < N) {
          S[j] = fmaf(exp_for<T>(dt * A[j]), S[j], dx * Bv[n]);
          y = fmaf(S[j], Cv[n], y);
        }
      }
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (lane == 0 && live) {
        const float z = s_z[tt * CB + cl];
        const float v = fmaf(Dc, xv, y);
        out[(size_t)(q0 + t0 + tt) * inner + c] = from_float<T>(v * (z / (1.0f + expf(-z))));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = lane + L * j;
    if (live && n < N) S_row[n] = S[j];
  }
}

template <typename T, int NS, int L>
int launch_selective_scan(const void* x, int inner, const void* z, long long z_stride, int z_col, const float* dbc,
                          long long dbc_stride, int R, int N, const float* w_dt, const float* b_dt, const float* A_log,
                          const float* Dv, float* state, long long state_stride, long long state_off, const int* cu_q,
                          const int* state_slots, void* out, int n_seqs, cudaStream_t stream) {
  constexpr int CB = kScanThreads / L;
  const size_t smem = sizeof(float) * kScanTokens * ((size_t)R + 2 * N + 3 * CB);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(selective_scan_kernel<T, NS, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_pdl(selective_scan_kernel<T, NS, L>, dim3((inner + CB - 1) / CB, n_seqs), dim3(kScanThreads), smem, stream,
                    (const T*)x, inner, (const T*)z, z_stride, z_col, dbc, dbc_stride, R, N, w_dt, b_dt, A_log, Dv, state,
                    state_stride, state_off, cu_q, state_slots, (T*)out);
}

template <typename T>
int pick_selective_scan(const void* x, int inner, const void* z, long long z_stride, int z_col, const float* dbc,
                        long long dbc_stride, int R, int N, const float* w_dt, const float* b_dt, const float* A_log,
                        const float* Dv, float* state, long long state_stride, long long state_off, const int* cu_q,
                        const int* state_slots, void* out, int n_seqs, cudaStream_t stream) {
#define TM_SCAN(NS_, L_)                                                                                                   \
  return launch_selective_scan<T, NS_, L_>(x, inner, z, z_stride, z_col, dbc, dbc_stride, R, N, w_dt, b_dt, A_log, Dv, state, \
                                           state_stride, state_off, cu_q, state_slots, out, n_seqs, stream)
  if (N <= 8) TM_SCAN(2, 4);
  if (N <= 16) TM_SCAN(4, 4);
  if (N <= 32) TM_SCAN(8, 4);
  if (N <= 64) TM_SCAN(16, 4);
  if (N <= 128) TM_SCAN(8, 16);
  if (N <= 256) TM_SCAN(16, 16);
#undef TM_SCAN
  return TM_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace tmk

// x [T, inner] and out [T, inner] in the activation dtype; z: token t's gate at z + t * z_stride + z_col; dbc: token t's
// [low (R) | B (N) | C (N)] at dbc + t * dbc_stride, float; w_dt [inner, R], b_dt [inner], A_log [inner, N], D [inner] float;
// a request's states [inner, N] start state_off floats into its slot of `state`.
extern "C" int tm_selective_scan(int dtype, const void* x, int inner, const void* z, long long z_stride, int z_col, const float* dbc,
                                 long long dbc_stride, int R, int N, const float* w_dt, const float* b_dt, const float* A_log,
                                 const float* Dv, float* state, long long state_stride, long long state_off, const int* cu_q,
                                 const int* state_slots, void* out, int n_seqs, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (inner < 1 || N < 1 || R < 1) return TM_ERR_UNSUPPORTED_SHAPE;
  if (dtype == TM_DTYPE_F32)
    return tmk::pick_selective_scan<float>(x, inner, z, z_stride, z_col, dbc, dbc_stride, R, N, w_dt, b_dt, A_log, Dv, state,
                                           state_stride, state_off, cu_q, state_slots, out, n_seqs, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::pick_selective_scan<__nv_bfloat16>(x, inner, z, z_stride, z_col, dbc, dbc_stride, R, N, w_dt, b_dt, A_log, Dv,
                                                   state, state_stride, state_off, cu_q, state_slots, out, n_seqs, stream);
  return TM_ERR_BAD_DTYPE;
}
