// Pieces of feed-forward layers beyond SwiGLU: the squared-relu activation, the router of a mixture of experts, the
// gated activation of all experts at once with the routing weight folded in, and a batched 32-bit matrix product.
//
// tm_moe_topk, one warp per token over the router's 32-bit logits (a matrix product made before it): the `top`
// largest are chosen (lowest index first among equals); their weights are the softmax over the chosen logits alone.
// Outputs: the chosen experts and weights ([T, top]) and a dense row of weights ([T, E], zero where not chosen).
//
// tm_glu_routed: gu [T, E, 2, F] (per expert: gate rows, then up rows) -> act [T, E, F] = silu(gate) * up * weight[t, e],
// exactly zero for experts the token did not choose (their products are never looked at), so that ONE matrix product
// of act with the experts' down matrices laid side by side along K gives the weighted sum of the chosen experts.
//
// tm_moe_choose: a router that scores every output with a softmax over ALL of them, s = softmax(z), chooses by
// s + correction (a learned vector that does not enter the weights), may restrict the choice to the best `keep` of
// `groups` equal groups of neighbouring outputs (a group's score: its largest choice score; outputs of other groups
// count as minus infinity), and weighs the `top` chosen by their s divided by the sum of the chosen s (+ 1e-20). The last
// `identity` outputs have no expert behind them: their result is the token's input itself; their summed weight is
// written per token beside the dense row of weights.
//
// tm_act_routed: up [T, E, F] -> act [T, E, F] = act(up) * weight[t, e] (act: the square of relu), zero where not chosen.
#include "common.cuh"

namespace tmk {

template <typename T>
__global__ void __launch_bounds__(256) relu2_kernel(const T* __restrict__ in, T* __restrict__ out, long long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_float(in[i]), 0.f);
    out[i] = from_float<T>(v * v);
  }
}

// One warp per token over its E logits (32-bit, from a matrix product; `bias` is added here when given).
__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                       int* __restrict__ top_idx, float* __restrict__ top_w,
                                                       float* __restrict__ dense_w, int T_, int E, int top, long long ld,
                                                       int scoring) {
  extern __shared__ float sm[];               // per warp: E logits
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T_) return;
  float* logit = sm + warp * E;
  for (int e = lane; e < E; e += 32) {
    logit[e] = logits[(size_t)t * ld + e] + (bias ? bias[e] : 0.f);
    dense_w[(size_t)t * E + e] = 0.f;
  }
  __syncwarp();
  // `top` rounds of arg-max; a chosen logit is marked by -inf in the scratch copy.
  float best0 = 0.f, denom = 0.f;
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = logit[e];
      if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (k == 0) best0 = bv;
    // scoring 0: a softmax over the chosen logits; 1: each chosen logit's sigmoid as it is
    const float ex = scoring == 1 ? 1.0f / (1.0f + expf(-bv)) : expf(bv - best0);
    denom += ex;
    if (lane == 0) {
      top_idx[(size_t)t * top + k] = bi;
      top_w[(size_t)t * top + k] = ex;
      logit[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    for (int k = 0; k < top; ++k) {
      const float wv = scoring == 1 ? top_w[(size_t)t * top + k] : top_w[(size_t)t * top + k] / denom;
      top_w[(size_t)t * top + k] = wv;
      dense_w[(size_t)t * E + top_idx[(size_t)t * top + k]] = wv;
    }
  }
}

// One warp per token over its n = experts + identity logits (32-bit). Ties go to the lowest index, in groups and outputs.
__global__ void __launch_bounds__(128) moe_choose_kernel(const float* __restrict__ logits, const float* __restrict__ correction,
                                                         int* __restrict__ top_idx, float* __restrict__ top_w,
                                                         float* __restrict__ dense_w, float* __restrict__ identity_w, int T_,
                                                         int n, int top, int groups, int keep, int identity) {
  extern __shared__ float sm[];               // per warp: n scores, n choice scores, `groups` group scores
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T_) return;
  float* score = sm + (size_t)warp * (2 * n + groups);
  float* choice = score + n;
  float* gscore = choice + n;
  float mx = -INFINITY;
  for (int e = lane; e < n; e += 32) {
    const float v = logits[(size_t)t * n + e];
    score[e] = v;
    mx = fmaxf(mx, v);
    dense_w[(size_t)t * n + e] = 0.f;
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < n; e += 32) {
    const float ex = expf(score[e] - mx);
    score[e] = ex;
    sum += ex;
  }
  sum = warp_sum(sum);
  for (int e = lane; e < n; e += 32) {
    score[e] = score[e] / sum;
    choice[e] = score[e] + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = n / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, choice[e]);
      gscore[g] = best;
    }
    __syncwarp();
    // `keep` rounds of arg-max over the groups; a kept group is marked by +inf, the others are closed afterwards
    for (int k = 0; k < keep; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gscore[g];
        if (v != INFINITY && (v > bv || (v == bv && g < bi) || bi == 0x7fffffff)) { bv = v; bi = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
      }
      if (lane == 0 && bi != 0x7fffffff) gscore[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  // `top` rounds of arg-max over the choice scores; a chosen output is marked by NaN in the scratch copy
  float denom = 0.f;
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < n; e += 32) {
      const float v = choice[e];
      if (v != v) continue;
      if (bi == 0x7fffffff || v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    const float sv = score[bi];
    denom += sv;
    if (lane == 0) {
      top_idx[(size_t)t * top + k] = bi;
      top_w[(size_t)t * top + k] = sv;
      choice[bi] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  if (lane == 0) {
    float idw = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = top_idx[(size_t)t * top + k];
      const float wv = top_w[(size_t)t * top + k] / (denom + 1e-20f);
      top_w[(size_t)t * top + k] = wv;
      dense_w[(size_t)t * n + e] = wv;
      if (e >= n - identity) idw += wv;
    }
    if (identity_w) identity_w[t] = idw;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) act_routed_kernel(const T* __restrict__ up, const float* __restrict__ dense_w,
                                                         int dense_stride, T* __restrict__ act, int E, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, e = blockIdx.y;
  const float wv = dense_w[(size_t)t * dense_stride + e];
  const T* u = up + ((size_t)t * E + e) * F;
  T* o = act + ((size_t)t * E + e) * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    float v = 0.f;
    if (wv != 0.f) {
      const float r = fmaxf(to_float(u[i]), 0.f);
      v = r * r * wv;
    }
    o[i] = from_float<T>(v);
  }
}

// out[t] += w[t] * x[t], row by row (the share of router outputs whose result is the input itself).
template <typename T>
__global__ void __launch_bounds__(256) add_scaled_rows_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                              const float* __restrict__ w, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float wv = w[t];
  if (wv == 0.f) return;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)t * H + i] = from_float<T>(fmaf(wv, to_float(x[(size_t)t * H + i]), to_float(out[(size_t)t * H + i])));
}

// Experts whose weight multiplies their INPUT: expert(w h) = W_down (silu(w g) * (w u)) with g = W_gate h, u = W_up h,
// so the two products run on h itself and the weight enters here (exact zeros for experts not chosen). Block
// (token, expert); expert number E is a shared expert of Fs numbers that every token uses, its output times
// sigmoid(shared_logit[t]). A token's row of gu is [E x (gate F | up F) | shared gate Fs | shared up Fs], of act
// [E x F | Fs].
template <typename T>
__global__ void __launch_bounds__(128) glu_routed_in_kernel(const T* __restrict__ gu, const float* __restrict__ dense_w,
                                                            T* __restrict__ act, int E, int F, int Fs,
                                                            const float* __restrict__ shared_logit, long long shared_ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, e = blockIdx.y;
  const size_t in_row = (size_t)E * 2 * F + 2 * (size_t)Fs, out_row = (size_t)E * F + Fs;
  if (e == E) {
    const float sg = shared_logit ? 1.0f / (1.0f + expf(-shared_logit[(size_t)t * shared_ld])) : 1.0f;
    const T* g = gu + (size_t)t * in_row + (size_t)E * 2 * F;
    T* o = act + (size_t)t * out_row + (size_t)E * F;
    for (int i = threadIdx.x; i < Fs; i += blockDim.x) {
      const float gv = to_float(g[i]);
      o[i] = from_float<T>(gv / (1.0f + expf(-gv)) * to_float(g[Fs + i]) * sg);
    }
    return;
  }
  const float wv = dense_w[(size_t)t * E + e];
  const T* g = gu + (size_t)t * in_row + (size_t)e * 2 * F;
  T* o = act + (size_t)t * out_row + (size_t)e * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    float v = 0.f;
    if (wv != 0.f) {
      const float gv = wv * to_float(g[i]);
      v = gv / (1.0f + expf(-gv)) * (wv * to_float(g[F + i]));
    }
    o[i] = from_float<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) glu_routed_kernel(const T* __restrict__ gu, const float* __restrict__ dense_w,
                                                         T* __restrict__ act, int E, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, e = blockIdx.y;
  const float wv = dense_w[(size_t)t * E + e];
  const T* g = gu + ((size_t)t * E + e) * 2 * F;
  T* o = act + ((size_t)t * E + e) * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    float v = 0.f;
    if (wv != 0.f) {
      const float gv = to_float(g[i]);
      v = gv / (1.0f + expf(-gv)) * to_float(g[F + i]) * wv;
    }
    o[i] = from_float<T>(v);
  }
}

// C[b][M, N] = A[b][M, K] . W[b][N, K]^T, 32-bit, every output element one accumulator walking k in order.
constexpr int GB = 32, GK = 16;
__global__ void __launch_bounds__(256) gemm_f32_nt_batched_kernel(const float* __restrict__ A, long long a_batch, int lda,
                                                                  const float* __restrict__ W, long long w_batch,
                                                                  float* __restrict__ C, long long c_batch, int ldc, int M,
                                                                  int N, int K) {
  __shared__ float As[GK][GB + 1];
  __shared__ float Ws[GK][GB + 1];
  A += (size_t)blockIdx.z * a_batch;
  W += (size_t)blockIdx.z * w_batch;
  C += (size_t)blockIdx.z * c_batch;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * GB, n0 = blockIdx.x * GB;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  const int lc = tid & 15, lr = tid >> 4;
  for (int k0 = 0; k0 < K; k0 += GK) {
    const int k = k0 + lc;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = lr + 16 * i;
      As[lc][r] = (m0 + r < M && k < K) ? A[(size_t)(m0 + r) * lda + k] : 0.f;
      Ws[lc][r] = (n0 + r < N && k < K) ? W[(size_t)(n0 + r) * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1], w0 = Ws[kk][tx * 2], w1 = Ws[kk][tx * 2 + 1];
      acc[0][0] = fmaf(a0, w0, acc[0][0]);
      acc[0][1] = fmaf(a0, w1, acc[0][1]);
      acc[1][0] = fmaf(a1, w0, acc[1][0]);
      acc[1][1] = fmaf(a1, w1, acc[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int m = m0 + ty * 2 + i, n = n0 + tx * 2 + j;
      if (m < M && n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
}

}  // namespace tmk

extern "C" int tm_relu2(int dtype, const void* in, void* out, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::relu2_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)in,
                           (float*)out, total);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::relu2_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream,
                           (const __nv_bfloat16*)in, (__nv_bfloat16*)out, total);
  return TM_ERR_BAD_DTYPE;
}

// logits [T, E] float (bias [E] float added when given); top_idx [T, top] int; top_w [T, top], dense_w [T, E] float.
extern "C" int tm_moe_topk(const float* logits, const float* bias, int* top_idx, float* top_w, float* dense_w, int T,
                           int E, int top, long long ld, int scoring, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top < 1 || top > E || E > 2048 || ld < E || (scoring != 0 && scoring != 1)) return TM_ERR_UNSUPPORTED_SHAPE;
  const int warps = 4;
  return tmk::launch_pdl(tmk::moe_topk_kernel, dim3((T + warps - 1) / warps), dim3(warps * 32),
                         (size_t)warps * E * sizeof(float), stream, logits, bias, top_idx, top_w, dense_w, T, E, top, ld,
                         scoring);
}

// gu [T, E * 2 F + 2 Fs], act [T, E F + Fs] dtype; dense_w [T, E] float; shared_logit: float, token t's at
// shared_logit[t * shared_ld] (null with Fs > 0: the shared expert is not gated).
extern "C" int tm_glu_routed_in(int dtype, const void* gu, const float* dense_w, void* act, int T, int E, int F, int Fs,
                                const float* shared_logit, long long shared_ld, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 65534 || E < 1 || F < 1 || Fs < 0) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid(T, E + (Fs > 0 ? 1 : 0));
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::glu_routed_in_kernel<float>, grid, dim3(128), 0, stream, (const float*)gu, dense_w,
                           (float*)act, E, F, Fs, shared_logit, shared_ld);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::glu_routed_in_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)gu,
                           dense_w, (__nv_bfloat16*)act, E, F, Fs, shared_logit, shared_ld);
  return TM_ERR_BAD_DTYPE;
}

// gu [T, E, 2, F], act [T, E, F] dtype; dense_w [T, E] float.
extern "C" int tm_glu_routed(int dtype, const void* gu, const float* dense_w, void* act, int T, int E, int F,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid(T, E);
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::glu_routed_kernel<float>, grid, dim3(128), 0, stream, (const float*)gu, dense_w,
                           (float*)act, E, F);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::glu_routed_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)gu,
                           dense_w, (__nv_bfloat16*)act, E, F);
  return TM_ERR_BAD_DTYPE;
}

// logits [T, n] float, n = experts + identity; correction [n] float or null; top_idx [T, top] int; top_w [T, top],
// dense_w [T, n] float; identity_w [T] float or null.
extern "C" int tm_moe_choose(const float* logits, const float* correction, int* top_idx, float* top_w, float* dense_w,
                             float* identity_w, int T, int n, int top, int groups, int keep, int identity, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top < 1 || top > n || n > 2048 || groups < 1 || n % groups || keep < 1 || keep > groups || identity < 0 || identity > n ||
      top > keep * (n / groups))
    return TM_ERR_UNSUPPORTED_SHAPE;
  const int warps = 4;
  return tmk::launch_pdl(tmk::moe_choose_kernel, dim3((T + warps - 1) / warps), dim3(warps * 32),
                         (size_t)warps * (2 * n + groups) * sizeof(float), stream, logits, correction, top_idx, top_w, dense_w,
                         identity_w, T, n, top, groups, keep, identity);
}

// up [T, E, F], act [T, E, F] dtype; dense_w float, token t's weights at dense_w + t * dense_stride.
extern "C" int tm_act_routed(int dtype, const void* up, const float* dense_w, int dense_stride, void* act, int T, int E, int F,
                             cudaStream_t stream) {
  if (T <= 0 || E <= 0) return 0;
  if (E > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid(T, E);
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::act_routed_kernel<float>, grid, dim3(128), 0, stream, (const float*)up, dense_w, dense_stride,
                           (float*)act, E, F);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::act_routed_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)up, dense_w,
                           dense_stride, (__nv_bfloat16*)act, E, F);
  return TM_ERR_BAD_DTYPE;
}

// out, x [T, H] dtype; w [T] float.
extern "C" int tm_add_scaled_rows(int dtype, void* out, const void* x, const float* w, int T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::add_scaled_rows_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)out, (const float*)x, w, H);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::add_scaled_rows_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out,
                           (const __nv_bfloat16*)x, w, H);
  return TM_ERR_BAD_DTYPE;
}

// A: batch b at A + b * a_batch, rows lda apart; W: [N, K] per batch, w_batch apart; C likewise with ldc.
extern "C" int tm_gemm_f32_nt_batched(const float* A, long long a_batch, int lda, const float* W, long long w_batch,
                                      float* C, long long c_batch, int ldc, int batches, int M, int N, int K,
                                      cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batches <= 0) return 0;
  if (K <= 0 || batches > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  const dim3 grid((N + tmk::GB - 1) / tmk::GB, (M + tmk::GB - 1) / tmk::GB, batches);
  if (grid.y > 65535) return TM_ERR_UNSUPPORTED_SHAPE;
  tmk::gemm_f32_nt_batched_kernel<<<grid, 256, 0, stream>>>(A, a_batch, lda, W, w_batch, C, c_batch, ldc, M, N, K);
  return tmk::launch_status();
}
