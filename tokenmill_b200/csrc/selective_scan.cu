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
// A block serves CB = 128 / L channels of one request; a channel's N states are dealt out over L lanes, NS = ceil(N / L)
// neighbouring states per lane in registers (state n on lane n / NS), so that a lane reads its B and C with 16-byte
// loads. The block keeps its channels' rows of W_dt in shared memory (row stride odd: no bank conflicts). Tokens are
// staged sixteen at a time: low, B and C (padded with zeros to NS * L), x, z, and the step sizes, which all threads
// compute together before the walk; a token's results wait in shared memory and leave together, gated, after the walk.
//
// Three ways to run (mode):
//   0  one walk over each request's tokens, from the slot's state and back into it. Whatever the cut of a sequence
//      into such steps, a state sees the same operations in the same order.
//   1  long portions, first pass: a block walks ONE time slice of slice_len tokens from a zero state and leaves the
//      slice's own state and, per channel, the sum of its step sizes in scratch memory. (The product of a slice's
//      decays is exp(A[c, n] * that sum).) tm_selective_pass_states then turns the scratch into every slice's state at
//      its start and the slot's state into the state after the last slice.
//   2  third pass: every slice again, from its start state, now with the outputs.
#include "common.cuh"

namespace tmk {

constexpr int kScanThreads = 128;
constexpr int kScanTokens = 16;
constexpr int kScanFew = 4;            // walks of fewer tokens read W_dt from global memory instead of staging it

// exp(x) to about one unit in the last place (1.05 at worst, a quarter on average): n = round(x / ln 2), r = x - n ln 2 with ln 2 in two pieces (the
// high one has enough trailing zero bits for n * high to be exact), a degree-7 polynomial on |r| <= 0.347 (remainder below
// 6e-9), then the exponent. Below -86 the result is 0. A decay is multiplied into a state once per token, so its error adds up
// over a sequence: the 32-bit run, whose logits are compared to a few units of 32-bit rounding, takes this form; the
// bfloat16 run takes the special-function unit (two units in the last place).
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

// The decay exp(dt * A) of one token. The 32-bit run keeps A and the careful exponential; the bfloat16 run keeps
// A * log2(e) and takes 2^x from the special-function unit.
template <typename T> __device__ __forceinline__ float decay_rate(float A) { return A * 1.4426950408889634f; }
template <> __device__ __forceinline__ float decay_rate<float>(float A) { return A; }
template <typename T> __device__ __forceinline__ float decay_of(float dt, float rate) { return exp2f(dt * rate); }
template <> __device__ __forceinline__ float decay_of<float>(float dt, float rate) { return exp_one_ulp(dt * rate); }

template <int NS> __device__ __forceinline__ void load_run(const float* p, float (&v)[NS]) {
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

template <typename T, int NS, int L, int MODE>
__global__ void __launch_bounds__(kScanThreads) selective_scan_kernel(
    const T* __restrict__ x, int inner, const T* __restrict__ zmat, long long z_stride, int z_col,
    const float* __restrict__ dbc, long long dbc_stride, int R, int N, const float* __restrict__ w_dt,
    const float* __restrict__ b_dt, const float* __restrict__ A_log, const float* __restrict__ Dv, float* __restrict__ state,
    long long state_stride, long long state_off, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
    T* __restrict__ out, int slice_len, int max_slices, float* __restrict__ slice_S, float* __restrict__ slice_dt) {
  constexpr int CB = kScanThreads / L;              // channels of a block
  constexpr int NP = NS * L;                        // states, padded
  extern __shared__ __align__(16) float smem[];
  const int RS = R | 1;
  float* s_B = smem;                                // [16][NP]
  float* s_C = s_B + kScanTokens * NP;              // [16][NP]
  float* s_x = s_C + kScanTokens * NP;              // [16][CB]
  float* s_z = s_x + kScanTokens * CB;              // [16][CB]
  float* s_dt = s_z + kScanTokens * CB;             // [16][CB]   the step sizes, then the walk's results
  float* s_low = s_dt + kScanTokens * CB;           // [16][R]
  float* s_w = s_low + kScanTokens * R;             // [CB][RS]
  float* s_b = s_w + CB * RS;                       // [CB] step-size bias, then [CB] D

  pdl_launch_dependents();
  pdl_wait();
  const int s = MODE == 0 ? blockIdx.y : blockIdx.y / max_slices;
  const int k = MODE == 0 ? 0 : blockIdx.y - s * max_slices;
  const int q_len = cu_q[s + 1] - cu_q[s];
  const int t_begin = MODE == 0 ? 0 : k * slice_len;
  const int t_end = MODE == 0 ? q_len : min(q_len, t_begin + slice_len);
  if (t_begin >= t_end) return;
  const int q0 = cu_q[s];
  const int c0 = blockIdx.x * CB;
  const int lane = threadIdx.x % L, cl = threadIdx.x / L;
  const int c = c0 + cl;
  const bool live = c < inner;
  float* S_row = MODE == 0 ? state + (size_t)state_slots[s] * state_stride + state_off + (size_t)(live ? c : 0) * N
                           : slice_S + ((size_t)blockIdx.y * inner + (live ? c : 0)) * N;

  // A walk of a few tokens (a decode step) does not stage its rows of W_dt: a channel's lanes share the rank-sized
  // product, each reading its part of the row from global memory.
  const bool few = MODE == 0 && q_len < kScanFew;
  if (!few) {
    for (int i = threadIdx.x; i < CB * R; i += kScanThreads) {
      const int cc = i / R, r = i - cc * R;
      s_w[cc * RS + r] = c0 + cc < inner ? w_dt[(size_t)(c0 + cc) * R + r] : 0.f;
    }
  }
  for (int i = threadIdx.x; i < CB; i += kScanThreads) {
    s_b[i] = c0 + i < inner ? b_dt[c0 + i] : 0.f;
    s_b[CB + i] = c0 + i < inner ? Dv[c0 + i] : 0.f;
  }

  float A[NS], S[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = lane * NS + j;
    const bool ok = live && n < N;
    A[j] = ok ? decay_rate<T>(-exp_for<T>(A_log[(size_t)c * N + n])) : 0.f;
    S[j] = (ok && MODE != 1) ? S_row[n] : 0.f;
  }
  float dt_sum = 0.f;

  for (int t0 = t_begin; t0 < t_end; t0 += kScanTokens) {
    const int nt = min(kScanTokens, t_end - t0);
    __syncthreads();                                // the previous tokens have left the staging
    for (int tt = threadIdx.x / 32; tt < nt; tt += kScanThreads / 32) {
      const float* row = dbc + (size_t)(q0 + t0 + tt) * dbc_stride;
      for (int i = threadIdx.x % 32; i < R; i += 32) s_low[tt * R + i] = row[i];
      for (int i = threadIdx.x % 32; i < NP; i += 32) {
        s_B[tt * NP + i] = i < N ? row[R + i] : 0.f;
        if (MODE != 1) s_C[tt * NP + i] = i < N ? row[R + N + i] : 0.f;
      }
      for (int i = threadIdx.x % 32; i < CB; i += 32) {
        const bool ok = c0 + i < inner;
        s_x[tt * CB + i] = ok ? to_float(x[(size_t)(q0 + t0 + tt) * inner + c0 + i]) : 0.f;
        if (MODE != 1) s_z[tt * CB + i] = ok ? to_float(zmat[(size_t)(q0 + t0 + tt) * z_stride + z_col + c0 + i]) : 0.f;
      }
    }
    __syncthreads();
    if (few) {
      const float* wr = w_dt + (size_t)(live ? c : 0) * R;
      for (int tt = 0; tt < nt; ++tt) {
        const float* low = s_low + tt * R;
        float acc = 0.f;
#pragma unroll 4
        for (int r = lane; r < R; r += L) acc = fmaf(wr[r], low[r], acc);
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) s_dt[tt * CB + cl] = live ? softplus32<T>(acc + s_b[cl]) : 0.f;
      }
    } else {
      // A thread takes one channel and TPT tokens, so that a number of its row of W_dt serves TPT products; every sum
      // still runs over the ranks in order. (Rows of tokens past nt hold old numbers; their sums are dropped.)
      constexpr int TPT = kScanTokens * CB / kScanThreads;
      const int cc = threadIdx.x % CB, tg = threadIdx.x / CB;
      const float* wr = s_w + cc * RS;
      const float* low = s_low + tg * TPT * R;
      float acc[TPT];
#pragma unroll
      for (int j = 0; j < TPT; ++j) acc[j] = 0.f;
      if ((R & 3) == 0) {
        for (int r = 0; r < R; r += 4) {
          const float w0 = wr[r], w1 = wr[r + 1], w2 = wr[r + 2], w3 = wr[r + 3];
#pragma unroll
          for (int j = 0; j < TPT; ++j) {
            const float4 l = *reinterpret_cast<const float4*>(low + j * R + r);
            acc[j] = fmaf(w0, l.x, acc[j]);
            acc[j] = fmaf(w1, l.y, acc[j]);
            acc[j] = fmaf(w2, l.z, acc[j]);
            acc[j] = fmaf(w3, l.w, acc[j]);
          }
        }
      } else {
        for (int r = 0; r < R; ++r) {
          const float wv = wr[r];
#pragma unroll
          for (int j = 0; j < TPT; ++j) acc[j] = fmaf(wv, low[j * R + r], acc[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < TPT; ++j) {
        const int tt = tg * TPT + j;
        if (tt < nt) s_dt[tt * CB + cc] = c0 + cc < inner ? softplus32<T>(acc[j] + s_b[cc]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = s_dt[tt * CB + cl], xv = s_x[tt * CB + cl];
      const float dx = dt * xv;
      float Bv[NS], Cv[NS];
      load_run<NS>(s_B + tt * NP + lane * NS, Bv);
      if (MODE != 1) load_run<NS>(s_C + tt * NP + lane * NS, Cv);
      float y = 0.f;
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        S[j] = fmaf(decay_of<T>(dt, A[j]), S[j], dx * Bv[j]);
        if (MODE != 1) y = fmaf(S[j], Cv[j], y);
      }
      if (MODE == 1) {
        dt_sum += dt;
      } else {
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        if (lane == 0) s_dt[tt * CB + cl] = y;      // (its lanes, all in this warp, have read the step size)
      }
    }
    if (MODE != 1) {
      __syncthreads();
      for (int i = threadIdx.x; i < nt * CB; i += kScanThreads) {
        const int tt = i / CB, cc = i - tt * CB;
        if (c0 + cc < inner) {
          const float z = s_z[i];
          const float v = fmaf(s_b[CB + cc], s_x[i], s_dt[i]);
          out[(size_t)(q0 + t0 + tt) * inner + c0 + cc] = from_float<T>(v * (z / (1.0f + expf(-z))));
        }
      }
    }
  }
  if (MODE != 2) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int n = lane * NS + j;
      if (live && n < N) S_row[n] = S[j];
    }
  }
  if (MODE == 1 && lane == 0 && live) slice_dt[(size_t)blockIdx.y * inner + c] = dt_sum;
}

// One thread per (request, channel, state): slice k's scratch state becomes the state at its start, and the slot's
// state the one after the last slice: S <- exp(A * sum of the slice's step sizes) S + the slice's own state.
template <typename T>
__global__ void __launch_bounds__(256) selective_pass_states_kernel(
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, const float* __restrict__ A_log, float* __restrict__ slice_S,
    const float* __restrict__ slice_dt, int inner, int N, int slice_len, int max_slices) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int q_len = cu_q[s + 1] - cu_q[s];
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)inner * N || q_len <= 0) return;
  const int c = (int)(e / N);
  const float rate = decay_rate<T>(-exp_for<T>(A_log[e]));
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off + e;
  float S = *slot;
  const int slices = (q_len + slice_len - 1) / slice_len;
  for (int k = 0; k < slices; ++k) {
    const size_t at = (size_t)s * max_slices + k;
    float* mine = slice_S + at * inner * N + e;
    const float own = *mine;
    *mine = S;
    S = fmaf(decay_of<T>(slice_dt[at * inner + c], rate), S, own);
  }
  *slot = S;
}

template <typename T, int NS, int L>
int launch_selective_scan(const void* x, int inner, const void* z, long long z_stride, int z_col, const float* dbc,
                          long long dbc_stride, int R, int N, const float* w_dt, const float* b_dt, const float* A_log,
                          const float* Dv, float* state, long long state_stride, long long state_off, const int* cu_q,
                          const int* state_slots, void* out, int n_seqs, int mode, int slice_len, int max_slices,
                          float* slice_S, float* slice_dt, cudaStream_t stream) {
  constexpr int CB = kScanThreads / L;
  const size_t smem = sizeof(float) * (kScanTokens * ((size_t)R + 2 * NS * L + 3 * CB) + (size_t)CB * (R | 1) + 2 * CB);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
#define TM_SCAN_MODE(M_)                                                                                                     \
  {                                                                                                                          \
    if (smem > 40 * 1024) {                                                                                                  \
      cudaError_t e = cudaFuncSetAttribute(selective_scan_kernel<T, NS, L, M_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                                       \
      if (e != cudaSuccess) return (int)e;                                                                                   \
    }                                                                                                                        \
    return launch_pdl(selective_scan_kernel<T, NS, L, M_>, dim3((inner + CB - 1) / CB, n_seqs * (M_ == 0 ? 1 : max_slices)), \
                      dim3(kScanThreads), smem, stream, (const T*)x, inner, (const T*)z, z_stride, z_col, dbc, dbc_stride, R, \
                      N, w_dt, b_dt, A_log, Dv, state, state_stride, state_off, cu_q, state_slots, (T*)out, slice_len,       \
                      max_slices, slice_S, slice_dt);                                                                        \
  }
  if (mode == 0) TM_SCAN_MODE(0)
  if (mode == 1) TM_SCAN_MODE(1)
  TM_SCAN_MODE(2)
#undef TM_SCAN_MODE
}

template <typename T>
int pick_selective_scan(const void* x, int inner, const void* z, long long z_stride, int z_col, const float* dbc,
                        long long dbc_stride, int R, int N, const float* w_dt, const float* b_dt, const float* A_log,
                        const float* Dv, float* state, long long state_stride, long long state_off, const int* cu_q,
                        const int* state_slots, void* out, int n_seqs, int mode, int slice_len, int max_slices,
                        float* slice_S, float* slice_dt, cudaStream_t stream) {
#define TM_SCAN(NS_, L_)                                                                                                   \
  return launch_selective_scan<T, NS_, L_>(x, inner, z, z_stride, z_col, dbc, dbc_stride, R, N, w_dt, b_dt, A_log, Dv, state, \
                                           state_stride, state_off, cu_q, state_slots, out, n_seqs, mode, slice_len,         \
                                           max_slices, slice_S, slice_dt, stream)
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
// a request's states [inner, N] start state_off floats into its slot of `state`. mode 0: one walk per request. modes 1
// and 2: the first and third pass over time slices of slice_len tokens, max_slices per request, through slice_S
// [n_seqs * max_slices, inner, N] and slice_dt [n_seqs * max_slices, inner] (float), with tm_selective_pass_states between.
extern "C" int tm_selective_scan(int dtype, const void* x, int inner, const void* z, long long z_stride, int z_col, const float* dbc,
                                 long long dbc_stride, int R, int N, const float* w_dt, const float* b_dt, const float* A_log,
                                 const float* Dv, float* state, long long state_stride, long long state_off, const int* cu_q,
                                 const int* state_slots, void* out, int n_seqs, int mode, int slice_len, int max_slices,
                                 float* slice_S, float* slice_dt, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (inner < 1 || N < 1 || R < 1 || mode < 0 || mode > 2) return TM_ERR_UNSUPPORTED_SHAPE;
  if (mode != 0 && (slice_len < 1 || max_slices < 1 || !slice_S || !slice_dt)) return TM_ERR_SCRATCH_TOO_SMALL;
  if (dtype == TM_DTYPE_F32)
    return tmk::pick_selective_scan<float>(x, inner, z, z_stride, z_col, dbc, dbc_stride, R, N, w_dt, b_dt, A_log, Dv, state,
                                           state_stride, state_off, cu_q, state_slots, out, n_seqs, mode, slice_len, max_slices,
                                           slice_S, slice_dt, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::pick_selective_scan<__nv_bfloat16>(x, inner, z, z_stride, z_col, dbc, dbc_stride, R, N, w_dt, b_dt, A_log, Dv,
                                                   state, state_stride, state_off, cu_q, state_slots, out, n_seqs, mode,
                                                   slice_len, max_slices, slice_S, slice_dt, stream);
  return TM_ERR_BAD_DTYPE;
}

// Between the two passes over time slices (see the top of the file). dtype chooses the same exponential as the scan's.
extern "C" int tm_selective_pass_states(int dtype, float* state, long long state_stride, long long state_off, const int* cu_q,
                                        const int* state_slots, const float* A_log, float* slice_S, const float* slice_dt,
                                        int n_seqs, int inner, int N, int slice_len, int max_slices, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (inner < 1 || N < 1 || slice_len < 1 || max_slices < 1 || !slice_S || !slice_dt) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid((unsigned)(((long long)inner * N + 255) / 256), n_seqs);
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::selective_pass_states_kernel<float>, grid, dim3(256), 0, stream, state, state_stride, state_off,
                           cu_q, state_slots, A_log, slice_S, slice_dt, inner, N, slice_len, max_slices);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::selective_pass_states_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, state, state_stride,
                           state_off, cu_q, state_slots, A_log, slice_S, slice_dt, inner, N, slice_len, max_slices);
  return TM_ERR_BAD_DTYPE;
}
