// A residual of several streams (hyper-connections) behind a norm, and the cap on the logits.
//
// tm_stream_norm, one block per row. The residual of a token is S streams of H numbers, [T, S, H] in 32-bit. In one pass
// over the row the kernel
//   * starts the streams, every one as table[id] * table_scale + pos_table[position] (32-bit), when ids are given;
//   * or takes in the previous sublayer's result y = branch + row_scale * branch2 (each optional):
//     x_t <- sum_s mix[s, t] x_s + out[t] y, all streams from the old ones (mix null: x_t <- x_t + y);
//   * reads the streams as u = sum_s in[s] x_s (in null: the plain sum);
//   * writes norm(u): Dynamic Tanh, tanh(alpha u) w + b, which needs no statistic of the row, or an RMS norm,
//     u / sqrt(mean(u^2) + eps) * w.
// With `rows` only those rows are read and normed, and the residual is left as it is (the model's last norm). S = 1
// with no mix is the ordinary residual stream. Everything is 32-bit; the output is rounded once.
//
// tm_softcap: x <- cap * tanh(scale x / cap) in place (32-bit logits); cap 0: x <- scale x.
#include "common.cuh"

namespace tmk {

constexpr int kMaxStreams = 8;

// W consecutive elements per access (W = 4: 16 bytes of float, 8 of bfloat16; the pointer must be aligned so).
template <int W, typename T> __device__ __forceinline__ void ldw(const T* p, float (&v)[W]) {
  if constexpr (W == 4) load4(p, v);
  else v[0] = to_float(p[0]);
}
template <int W, typename T> __device__ __forceinline__ void stw(T* p, const float (&v)[W]) {
  if constexpr (W == 4) store4(p, v);
  else p[0] = from_float<T>(v[0]);
}

// SC: the number of streams when it is 1 to 4 (loops unrolled without tests), 0 for any number up to kMaxStreams.
// W: elements per thread and access in the first pass over the row.
template <typename T, int SC, int W>
__global__ void __launch_bounds__(256) stream_norm_kernel(
    float* __restrict__ resid, int S, int H, const int* __restrict__ ids, const T* __restrict__ table,
    const int* __restrict__ positions, const T* __restrict__ pos_table, const T* __restrict__ branch,
    const T* __restrict__ branch2, const float* __restrict__ row_scale, long long row_scale_stride,
    const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ in_w,
    const int* __restrict__ rows, int mode, const float* __restrict__ alpha_p, const float* __restrict__ w,
    const float* __restrict__ b, float eps, T* __restrict__ out, float table_scale) {
  constexpr int NS = SC ? SC : kMaxStreams;
  __shared__ float red[32];
  __shared__ float coef[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* x = resid + (size_t)t * S * H;
  float* m_s = coef;                                  // [from][to]
  float* o_s = coef + kMaxStreams * kMaxStreams;
  float* i_s = o_s + kMaxStreams;
  if (threadIdx.x < S * S) m_s[threadIdx.x] = mix ? mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    o_s[threadIdx.x] = out_w ? out_w[threadIdx.x] : 1.f;
    i_s[threadIdx.x] = in_w ? in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const bool start = ids != nullptr;
  const bool takes = branch != nullptr || branch2 != nullptr;
  const float rs = row_scale ? row_scale[(size_t)t * row_scale_stride] : 1.f;
  const T* e_row = start ? table + (size_t)ids[t] * H : nullptr;
  const T* p_row = (start && pos_table) ? pos_table + (size_t)positions[t] * H : nullptr;
  const float alpha = mode == 0 ? alpha_p[0] : 0.f;
  T* o_row = out + (size_t)r * H;

  float sq = 0.f;
  for (int i = threadIdx.x * W; i < H; i += blockDim.x * W) {
    float xs[NS][W];
    if (start) {
      float v[W];
      ldw<W>(e_row + i, v);
#pragma unroll
      for (int e = 0; e < W; ++e) v[e] *= table_scale;
      if (p_row) {
        float pv[W];
        ldw<W>(p_row + i, pv);
#pragma unroll
        for (int e = 0; e < W; ++e) v[e] += pv[e];
      }
#pragma unroll
      for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int e = 0; e < W; ++e) xs[s][e] = v[e];
    } else {
#pragma unroll
      for (int s = 0; s < NS; ++s)
        if (SC || s < S) ldw<W>(x + (size_t)s * H + i, xs[s]);
    }
    if (takes) {
      float y[W];
#pragma unroll
      for (int e = 0; e < W; ++e) y[e] = 0.f;
      if (branch) ldw<W>(branch + (size_t)t * H + i, y);
      if (branch2) {
        float y2[W];
        ldw<W>(branch2 + (size_t)t * H + i, y2);
#pragma unroll
        for (int e = 0; e < W; ++e) y[e] = fmaf(rs, y2[e], y[e]);
      }
      float nx[NS][W];
#pragma unroll
      for (int to = 0; to < NS; ++to) {
        if (!SC && to >= S) continue;
#pragma unroll
        for (int e = 0; e < W; ++e) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < NS; ++s)
            if (SC || s < S) acc = fmaf(m_s[s * S + to], xs[s][e], acc);
          nx[to][e] = fmaf(o_s[to], y[e], acc);
        }
      }
#pragma unroll
      for (int s = 0; s < NS; ++s)
        if (SC || s < S) {
#pragma unroll
          for (int e = 0; e < W; ++e) xs[s][e] = nx[s][e];
        }
    }
    if (!rows && (start || takes)) {
#pragma unroll
      for (int s = 0; s < NS; ++s)
        if (SC || s < S) stw<W>(x + (size_t)s * H + i, xs[s]);
    }
    float u[W];
#pragma unroll
    for (int e = 0; e < W; ++e) {
      u[e] = 0.f;
#pragma unroll
      for (int s = 0; s < NS; ++s)
        if (SC || s < S) u[e] = fmaf(i_s[s], xs[s][e], u[e]);
    }
    if (mode == 0) {
      float wv[W], o[W];
      ldw<W>(w + i, wv);
#pragma unroll
      for (int e = 0; e < W; ++e) o[e] = 0.f;
      if (b) ldw<W>(b + i, o);
#pragma unroll
      for (int e = 0; e < W; ++e) o[e] = fmaf(tanhf(alpha * u[e]), wv[e], o[e]);
      stw<W>(o_row + i, o);
    } else {
#pragma unroll
      for (int e = 0; e < W; ++e) sq = fmaf(u[e], u[e], sq);       // the RMS form needs the whole row's sum first: u is computed again below
    }
  }
  if (mode == 0) return;
  const float inv = 1.0f / sqrtf(block_sum(sq, red) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    // the streams are final now: in the residual for an updating pass, or recomputed for a gathered read-only row
    float u = 0.f;
    if (rows && (start || takes)) {
      // (the last norm of a model: read-only; recompute as above)
      float xs[kMaxStreams];
      if (start) {
        float v = to_float(e_row[i]) * table_scale;
        if (p_row) v += to_float(p_row[i]);
        for (int s = 0; s < S; ++s) xs[s] = v;
      } else {
        for (int s = 0; s < S; ++s) xs[s] = x[(size_t)s * H + i];
      }
      if (takes) {
        float y = branch ? to_float(branch[(size_t)t * H + i]) : 0.f;
        if (branch2) y = fmaf(rs, to_float(branch2[(size_t)t * H + i]), y);
        for (int to = 0; to < S; ++to) {
          float acc = 0.f;
          for (int s = 0; s < S; ++s) acc = fmaf(m_s[s * S + to], xs[s], acc);
          u = fmaf(i_s[to], fmaf(o_s[to], y, acc), u);
        }
      } else {
        for (int s = 0; s < S; ++s) u = fmaf(i_s[s], xs[s], u);
      }
    } else {
      for (int s = 0; s < S; ++s) u = fmaf(i_s[s], x[(size_t)s * H + i], u);
    }
    o_row[i] = from_float<T>(u * inv * w[i]);
  }
}

__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ x, long long n, float cap, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float z = x[i] * scale;
  x[i] = cap > 0.f ? cap * tanhf(z / cap) : z;
}

template <typename T>
int launch_stream_norm(float* resid, int S, int H, const int* ids, const void* table, const int* positions, const void* pos_table,
                       const void* branch, const void* branch2, const float* row_scale, long long row_scale_stride,
                       const float* mix, const float* out_w, const float* in_w, const int* rows, int mode, const float* alpha,
                       const float* w, const float* b, float eps, void* out, int n_rows, float table_scale,
                       cudaStream_t stream) {
  // four elements per access where every row starts on 16 bytes
  const uintptr_t all = (uintptr_t)resid | (uintptr_t)table | (uintptr_t)pos_table | (uintptr_t)branch | (uintptr_t)branch2 |
                        (uintptr_t)w | (uintptr_t)b | (uintptr_t)out;
  const bool wide = !(H & 3) && !(all & 15);
#define TM_STREAMS(SC_, W_)                                                                                                  \
  return launch_pdl(stream_norm_kernel<T, SC_, W_>, dim3(n_rows), dim3(256), 0, stream, resid, S, H, ids, (const T*)table,   \
                    positions, (const T*)pos_table, (const T*)branch, (const T*)branch2, row_scale, row_scale_stride, mix,   \
                    out_w, in_w, rows, mode, alpha, w, b, eps, (T*)out, table_scale)
  if (wide) {
    if (S == 1) TM_STREAMS(1, 4);
    if (S == 2) TM_STREAMS(2, 4);
    if (S == 3) TM_STREAMS(3, 4);
    if (S == 4) TM_STREAMS(4, 4);
  }
  TM_STREAMS(0, 1);
#undef TM_STREAMS
}

}  // namespace tmk

// resid [T, S, H] float; ids [T] + table [vocab, H] (+ positions [T] + pos_table [n, H]) start the streams; branch, branch2
// [T, H] in the activation dtype, row_scale float (one per token, row_scale_stride apart); mix [S, S] ([from, to]), out_w [S],
// in_w [S] float or null; rows [n_rows] or null; mode 0: Dynamic Tanh (alpha: one float on the device, w, b [H], b may be null),
// mode 1: RMS (w [H], eps); out [n_rows, H].
extern "C" int tm_stream_norm(int dtype, float* resid, int S, int H, const int* ids, const void* table, const int* positions,
                              const void* pos_table, const void* branch, const void* branch2, const float* row_scale,
                              long long row_scale_stride, const float* mix, const float* out_w, const float* in_w, const int* rows,
                              int mode, const float* alpha, const float* w, const float* b, float eps, void* out, int n_rows,
                              float table_scale, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (S < 1 || S > tmk::kMaxStreams || H < 1 || (mode != 0 && mode != 1) || (mode == 0 && !alpha)) return TM_ERR_UNSUPPORTED_SHAPE;
  if (ids && (branch || branch2)) return TM_ERR_UNSUPPORTED_SHAPE;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_stream_norm<float>(resid, S, H, ids, table, positions, pos_table, branch, branch2, row_scale,
                                          row_scale_stride, mix, out_w, in_w, rows, mode, alpha, w, b, eps, out, n_rows, table_scale, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_stream_norm<__nv_bfloat16>(resid, S, H, ids, table, positions, pos_table, branch, branch2, row_scale,
                                                  row_scale_stride, mix, out_w, in_w, rows, mode, alpha, w, b, eps, out, n_rows,
                                                  table_scale, stream);
  return TM_ERR_BAD_DTYPE;
}

extern "C" int tm_softcap(float* x, long long n, float cap, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap >= 0.f)) return TM_ERR_UNSUPPORTED_SHAPE;
  return tmk::launch_pdl(tmk::softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap, scale);
}
