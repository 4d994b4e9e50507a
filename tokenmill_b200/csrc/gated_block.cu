// Kernels of a pre-norm block whose branches enter the stream through a learned gate and whose sublayers read their
// input through a short causal convolution, plus the small kernels its branches need. All arithmetic is 32-bit;
// every output is rounded once.
//
// tm_gated_add_rmsnorm, one block per row:
//   x = table[ids[row]] * table_scale                     (the stream starts here), or
//   x = resid[row] + sigmoid(gate[row] + gate_bias) * branch[row]      (gate absent: the branch is added as it is)
//   out[row] = x / sqrt(mean(x^2) + eps) * w
// `gate` is the gate's pre-activation as a 32-bit matrix product result. With `rows`, only those rows are normed,
// written densely, and the stream is left as it is.
//
// tm_canon_conv, one block per row: out[t] = h[t] + sum_j w[:, j] h[t - taps + 1 + j]. Rows before the step's first row
// of a request come from the request's state slot (its last taps - 1 inputs, oldest first; zeros for a new request).
// The block of a request's first row computes every row that still reads the slot (the first taps - 1 of the step) and
// then writes the step's last taps - 1 inputs back, a thread per channel doing both: nothing else touches the slot.
//
// tm_glu: out[t, i] = act(gu[t, i]) * gu[t, I + i], act = silu or the tanh form of gelu.
//
// tm_norm_pair_mean: out = (rmsnorm(a) wa + rmsnorm(b) wb) / 2, each row of a and b by its own root mean square.
//
// tm_head_norm_gate: y [T, heads, dv] float32 (first divided by den[T, heads], where given) -> each head divided by its
// root mean square, times weight, times sigmoid or silu of the gate's pre-activation read from a 32-bit product (or
// no gate).
#include "common.cuh"

namespace tmk {

template <typename T>
__global__ void __launch_bounds__(256) gated_add_rmsnorm_kernel(
    float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ gate, long long gate_stride,
    const float* __restrict__ gate_bias, const int* __restrict__ ids, const T* __restrict__ table, float table_scale,
    const int* __restrict__ rows, const float* __restrict__ w, float eps, T* __restrict__ out, int H) {
  extern __shared__ __align__(16) float xs[];  // H floats + 32 for the reduction
  float* red = xs + H;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const bool write_back = !rows && (ids || branch);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float x;
    if (ids) {
      x = to_float(table[(size_t)ids[src] * H + i]) * table_scale;
    } else {
      x = resid[(size_t)src * H + i];
      if (branch) {
        const float y = to_float(branch[(size_t)src * H + i]);
        if (gate) {
          const float z = gate[(size_t)src * gate_stride + i] + (gate_bias ? gate_bias[i] : 0.f);
          x += y / (1.0f + expf(-z));
        } else {
          x += y;
        }
      }
    }
    if (write_back) resid[(size_t)src * H + i] = x;
    xs[i] = x;
    ss += x * x;
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)r * H + i] = from_float<T>(xs[i] * rstd * w[i]);
}

constexpr int kMaxTaps = 16;

// TAPS > 0: the number of taps is known when compiling (every loop unrolls, the carried inputs sit in registers);
// TAPS == 0: any number up to kMaxTaps. `vec`: C is a multiple of 4 and a thread takes four channels per access.
template <typename T, int TAPS>
__global__ void __launch_bounds__(256) canon_conv_kernel(
    const T* __restrict__ h, const float* __restrict__ w, float* __restrict__ state, long long state_stride,
    const int* __restrict__ cu_q, const int* __restrict__ seq_of_token, const int* __restrict__ state_slots,
    T* __restrict__ out, int C, int taps_rt, int vec) {
  constexpr int MAXT = TAPS > 0 ? TAPS : kMaxTaps;
  const int taps = TAPS > 0 ? TAPS : taps_rt;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const int first = cu_q[s], end = cu_q[s + 1];
  const int local = t - first;
  const int carry = taps - 1;
  if (local >= carry) {                     // every tap lies inside the step
    if (vec) {
      for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
        float wv[4 * MAXT];                 // the four channels' weights lie side by side: 16 bytes per access
        if (TAPS > 0) {
#pragma unroll
          for (int i = 0; i < TAPS; ++i) {
            const float4 x = *reinterpret_cast<const float4*>(w + (size_t)c * TAPS + 4 * i);
            wv[4 * i] = x.x; wv[4 * i + 1] = x.y; wv[4 * i + 2] = x.z; wv[4 * i + 3] = x.w;
          }
        }
#pragma unroll
        for (int j = 0; j < MAXT; ++j) {
          if (j < taps) {
            load4(h + (size_t)(t - carry + j) * C + c, v);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              acc[e] = fmaf(TAPS > 0 ? wv[e * MAXT + j] : w[(size_t)(c + e) * taps + j], v[e], acc[e]);
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] += v[e];         // the last tap's input is h[t]
        store4(out + (size_t)t * C + c, acc);
      }
      return;
    }
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float acc = 0.f;
      for (int j = 0; j < taps; ++j) acc = fmaf(w[(size_t)c * taps + j], to_float(h[(size_t)(t - carry + j) * C + c]), acc);
      out[(size_t)t * C + c] = from_float<T>(to_float(h[(size_t)t * C + c]) + acc);
    }
    return;
  }
  if (local != 0) return;                   // the first row's block does these rows
  float* slot = state + (size_t)state_slots[s] * state_stride;
  const int n = end - first;
  const int head = min(n, carry);
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float old[MAXT], wt[MAXT], cur[MAXT];   // carried inputs, weights, the step's first inputs
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {
      old[j] = j < carry ? slot[(size_t)j * C + c] : 0.f;
      wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
      cur[j] = j < head ? to_float(h[(size_t)(first + j) * C + c]) : 0.f;
    }
#pragma unroll
    for (int r = 0; r < MAXT; ++r) {        // row first + r reads positions r - carry .. r of the step
      if (r < head) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < MAXT; ++j) {
          if (j < taps) {
            const int p = r - carry + j;    // p < 0: slot entry carry + p
            float v = 0.f;
#pragma unroll
            for (int i = 0; i < MAXT; ++i) {
              if (p < 0 && i == carry + p) v = old[i];
              if (p >= 0 && i == p) v = cur[i];
            }
            acc = fmaf(wt[j], v, acc);
          }
        }
        out[(size_t)(first + r) * C + c] = from_float<T>(cur[r] + acc);
      }
    }
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {        // the last `carry` inputs of (old inputs ++ this step's)
      if (j < carry) {
        const int p = n - carry + j;
        float v = 0.f;
        if (p >= head) {
          v = to_float(h[(size_t)(first + p) * C + c]);
        } else {
#pragma unroll
          for (int i = 0; i < MAXT; ++i) {
            if (p < 0 && i == carry + p) v = old[i];
            if (p >= 0 && i == p) v = cur[i];
          }
        }
        slot[(size_t)j * C + c] = v;
      }
    }
  }
}

// tanh as 1 - 2 / (exp(2x) + 1): absolute error of the order of 1e-7 in 32-bit
__device__ __forceinline__ float fast_tanh(float x) { return 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f); }

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.0f + fast_tanh(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <int ACT> __device__ __forceinline__ float glu_act(float g) {
  return ACT == 0 ? g / (1.0f + expf(-g)) : gelu_tanh(g);
}

template <typename T, int ACT>
__global__ void __launch_bounds__(256) glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  if (vec) {                                // I a multiple of 4: four elements per access
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (i >= I) return;
    float g[4], u[4];
    load4(gu + t * 2 * I + i, g);
    load4(gu + t * 2 * I + I + i, u);
#pragma unroll
    for (int e = 0; e < 4; ++e) g[e] = glu_act<ACT>(g[e]) * u[e];
    store4(out + t * I + i, g);
    return;
  }
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= I) return;
  out[t * I + i] = from_float<T>(glu_act<ACT>(to_float(gu[t * 2 * I + i])) * to_float(gu[t * 2 * I + I + i]));
}

template <typename T>
__global__ void __launch_bounds__(256) norm_pair_mean_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                             const float* __restrict__ wa, const float* __restrict__ wb,
                                                             float eps, T* __restrict__ out, int H, int vec) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * H;
  float sa = 0.f, sb = 0.f;
  if (vec) {                                // H a multiple of 4: four elements per access
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float x[4], y[4];
      load4(a + row + i, x);
      load4(b + row + i, y);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        sa += x[e] * x[e];
        sb += y[e] * y[e];
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float x = to_float(a[row + i]), y = to_float(b[row + i]);
      sa += x * x;
      sb += y * y;
    }
  }
  const float ra = 1.0f / sqrtf(block_sum(sa, red) / (float)H + eps);
  const float rb = 1.0f / sqrtf(block_sum(sb, red) / (float)H + eps);
  if (vec) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float x[4], y[4];
      load4(a + row + i, x);
      load4(b + row + i, y);
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = 0.5f * (x[e] * ra * wa[i + e] + y[e] * rb * wb[i + e]);
      store4(out + row + i, x);
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[row + i] = from_float<T>(0.5f * (to_float(a[row + i]) * ra * wa[i] + to_float(b[row + i]) * rb * wb[i]));
}

// out = sa a + sb b, elementwise in 32-bit, rounded once.
template <typename T>
__global__ void __launch_bounds__(256) weighted_pair_kernel(const T* __restrict__ a, const T* __restrict__ b, float sa, float sb,
                                                            T* __restrict__ out, long long n, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (vec ? 4 : 1);
  if (i0 >= n) return;
  if (vec) {
    float x[4], y[4];
    load4(a + i0, x);
    load4(b + i0, y);
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = fmaf(sa, x[e], sb * y[e]);
    store4(out + i0, x);
  } else {
    out[i0] = from_float<T>(fmaf(sa, to_float(a[i0]), sb * to_float(b[i0])));
  }
}

// The gate's factor from its pre-activation: sigmoid (act 0) or silu (act 1); no gate: 1.
__device__ __forceinline__ float gate_value(const float* gate, size_t at, int act) {
  if (!gate) return 1.0f;
  const float z = gate[at];
  const float sg = 1.0f / (1.0f + expf(-z));
  return act == 1 ? z * sg : sg;
}

// One warp per (row, head); heads of 512 numbers and more take head_norm_gate_block_kernel.
template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ y, const float* __restrict__ den,
                                                             const float* __restrict__ gate,
                                                             long long gate_stride, int gate_act, const float* __restrict__ w,
                                                             float eps, T* __restrict__ out, long long out_ld, int heads,
                                                             int dv, long long n_pairs) {
  pdl_launch_dependents();
  pdl_wait();
  const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= n_pairs) return;
  const int lane = threadIdx.x & 31;
  const long long t = pair / heads;
  const int hd = (int)(pair - t * heads);
  const float* src = y + (size_t)pair * dv;
  const float dn = den ? den[pair] : 1.f;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) {
    const float o = src[i] / dn;
    ss += o * o;
  }
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int i = lane; i < dv; i += 32) {
    const int c = hd * dv + i;
    out[(size_t)t * out_ld + c] = from_float<T>(src[i] / dn * rstd * w[c] * gate_value(gate, (size_t)t * gate_stride + c, gate_act));
  }
}

// One block per (row, head), for heads of many numbers (heads normed together count as one head).
template <typename T>
__global__ void __launch_bounds__(256) head_norm_gate_block_kernel(const float* __restrict__ y, const float* __restrict__ den,
                                                                   const float* __restrict__ gate, long long gate_stride,
                                                                   int gate_act, const float* __restrict__ w, float eps,
                                                                   T* __restrict__ out, long long out_ld, int heads, int dv) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const long long pair = blockIdx.x;
  const long long t = pair / heads;
  const int hd = (int)(pair - t * heads);
  const float* src = y + (size_t)pair * dv;
  const size_t g0 = (size_t)t * gate_stride + (size_t)hd * dv;
  const float dn = den ? den[pair] : 1.f;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dv; i += blockDim.x) {
    const float o = src[i] / dn;
    ss += o * o;
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)dv + eps);
  for (int i = threadIdx.x; i < dv; i += blockDim.x)
    out[(size_t)t * out_ld + (size_t)hd * dv + i] = from_float<T>(src[i] / dn * rstd * w[hd * dv + i] * gate_value(gate, g0 + i, gate_act));
}

}  // namespace tmk

using namespace tmk;

#define TM_BY_DTYPE(dtype, ...)                                              \
  if ((dtype) == TM_DTYPE_F32) { using T = float; __VA_ARGS__; }             \
  if ((dtype) == TM_DTYPE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }    \
  return TM_ERR_BAD_DTYPE;

// resid [T, H] float; branch [T, H] dtype or null; gate: float, row stride gate_stride, or null; gate_bias [H] float or
// null; ids [T] + table [V, H] dtype or null; rows [n_rows] or null; w [H] float; out [n_rows, H] dtype.
extern "C" int tm_gated_add_rmsnorm(int dtype, float* resid, const void* branch, const float* gate, long long gate_stride,
                                    const float* gate_bias, const int* ids, const void* table, float table_scale,
                                    const int* rows, const float* w, float eps, void* out, int n_rows, int H,
                                    cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  TM_BY_DTYPE(dtype, {
    auto kern = gated_add_rmsnorm_kernel<T>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(kern, dim3(n_rows), dim3(256), smem, stream, resid, (const T*)branch, gate, gate_stride, gate_bias,
                      ids, (const T*)table, table_scale, rows, w, eps, (T*)out, H);
  })
}

// h, out [T, C] dtype; w [C, taps] float; state: float, a request's slot starts at state + slot * state_stride and holds
// [taps - 1, C] there.
extern "C" int tm_canon_conv(int dtype, const void* h, const float* w, float* state, long long state_stride,
                             const int* cu_q, const int* seq_of_token, const int* state_slots, void* out, int T_rows, int C,
                             int taps, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (taps < 1 || taps > kMaxTaps) return TM_ERR_UNSUPPORTED_SHAPE;
  const int vec = C % 4 == 0;
#define TM_CANON(TT)                                                                                                   \
  return launch_pdl(canon_conv_kernel<T, TT>, dim3(T_rows), dim3(256), 0, stream, (const T*)h, w, state, state_stride, cu_q, \
                    seq_of_token, state_slots, (T*)out, C, taps, vec);
  TM_BY_DTYPE(dtype, {
    switch (taps) {
      case 1: TM_CANON(1) case 2: TM_CANON(2) case 3: TM_CANON(3) case 4: TM_CANON(4) case 5: TM_CANON(5) case 6: TM_CANON(6)
      case 7: TM_CANON(7) case 8: TM_CANON(8)
      default: TM_CANON(0)
    }
  })
#undef TM_CANON
}

// gu [T, 2 I] (gate columns first) -> out [T, I]; act 0: silu, 1: gelu (tanh form).
extern "C" int tm_glu(int dtype, int act, const void* gu, void* out, int T_rows, int I, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (act != 0 && act != 1) return TM_ERR_UNSUPPORTED_SHAPE;
  const int vec = I % 4 == 0;
  const dim3 grid(T_rows, vec ? (I / 4 + 255) / 256 : (I + 255) / 256);
  TM_BY_DTYPE(dtype, {
    if (act == 0) return launch_pdl(glu_kernel<T, 0>, grid, dim3(256), 0, stream, (const T*)gu, (T*)out, I, vec);
    return launch_pdl(glu_kernel<T, 1>, grid, dim3(256), 0, stream, (const T*)gu, (T*)out, I, vec);
  })
}

extern "C" int tm_norm_pair_mean(int dtype, const void* a, const void* b, const float* wa, const float* wb, float eps,
                                 void* out, int T_rows, int H, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  TM_BY_DTYPE(dtype, return launch_pdl(norm_pair_mean_kernel<T>, dim3(T_rows), dim3(256), 0, stream, (const T*)a,
                                       (const T*)b, wa, wb, eps, (T*)out, H, (int)(H % 4 == 0)))
}

// a, b, out: n numbers each; out = sa a + sb b.
extern "C" int tm_weighted_pair(int dtype, const void* a, const void* b, float sa, float sb, void* out, long long n,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  const int vec = n % 4 == 0 && !(((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15);
  const long long threads = vec ? n / 4 : n;
  TM_BY_DTYPE(dtype, return launch_pdl(weighted_pair_kernel<T>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream,
                                       (const T*)a, (const T*)b, sa, sb, (T*)out, n, vec))
}

// y [T, heads * dv] float; den [T, heads] float or null; gate: float pre-activations, element (t, c) at
// gate + t * gate_stride + c, through a sigmoid (gate_act 0) or silu (1), or null for no gate; w [heads * dv]; out:
// element (t, c) at out + t * out_ld + c.
extern "C" int tm_head_norm_gate(int dtype, const float* y, const float* den, const float* gate, long long gate_stride,
                                 int gate_act, const float* w, float eps, void* out, long long out_ld, int T_rows, int heads,
                                 int dv, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (gate_act != 0 && gate_act != 1) return TM_ERR_UNSUPPORTED_SHAPE;
  const long long pairs = (long long)T_rows * heads;
  if (dv >= 512) {
    TM_BY_DTYPE(dtype, return launch_pdl(head_norm_gate_block_kernel<T>, dim3((unsigned)pairs), dim3(256), 0, stream, y, den, gate,
                                         gate_stride, gate_act, w, eps, (T*)out, out_ld, heads, dv))
  }
  TM_BY_DTYPE(dtype, return launch_pdl(head_norm_gate_kernel<T>, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, stream, y,
                                       den, gate, gate_stride, gate_act, w, eps, (T*)out, out_ld, heads, dv, pairs))
}
