// Matrix memories whose decay is computed per token, and the small kernels in front of them.
//
// tm_gated_memory: per head a d x dv memory S, from the state the request's slot holds, walked token by token:
//   decay   per head and token one number g_t:            S <- g_t S
//           or per head, token and row a number f_t[r]:   S[r, :] <- f_t[r] S[r, :]   (the key is then k_t = 1 - f_t)
//   write   plain:       S <- S + k_t v_t^T
//           delta rule:  u = beta_t (v_t - S^T k_t), S <- S + k_t u^T      (after the decay)
//   read    o_t = S^T q_t                                  (after the write)
// q and k (or f) are column ranges (qk_heads x d) of one 32-bit matrix, v another (heads x dv); head h reads q/k head
// h / (heads / qk_heads). g and beta come as gb [T, 2 heads] (g first). Everything is 32-bit; o is written in 32-bit.
//
// One block of 256 threads per (tile of columns, head, request or time slice). Every column of S evolves on its own
// (the delta rule's correction S^T k is a sum down the column), so a column's d numbers are spread over `parts`
// neighbouring lanes, 16 rows each in registers (lane p takes rows 4 p .. 4 p + 3 of every group of 4 * parts rows),
// and both sums down a column end in shuffles among those lanes. A request's memories are laid out [heads][dv][d_pad],
// a column's rows side by side (d_pad = 16 * parts; rows >= d stay zero). Tokens pass through two shared-memory buffers
// of sixteen, filled by asynchronous copies while the other is walked strictly in order.
//
// Three ways to run (mode):
//   0  one walk over each request's tokens, from the slot's memory and back into it. A sequence may be cut anywhere.
//   1  long portions, first pass: a block walks ONE time slice of slice_len tokens from a zero memory (no q, no
//      results) and leaves the slice's own memory in scratch. What a slice does to the memory it starts from is linear:
//      S_end = P S_start + S_own. With row decays P is diagonal, the product of the slice's f per row: it is walked as
//      ONE more column that starts at 1 and is never written to. With the delta rule P = prod_t g_t (I - beta_t k_t
//      k_t^T) is a full d x d matrix: it is walked as d more columns that start as the identity with v = 0.
//      tm_gated_memory_pass_states then turns the scratch into every slice's memory at its start, one slice after the
//      other, and the slot's memory into the one after the last slice.
//   2  third pass: every slice again, from its start memory, now with the results.
//
// tm_short_conv_state: a causal convolution over time on every channel of a 32-bit projection (bias added first),
// y_t = act(sum_j w[:, j] u_(t - taps + 1 + j)), the last taps - 1 inputs of a request carried in its slot.
// tm_delta_prepare: q and k to unit length per head (q also times d^-1/2), beta = sigmoid(.), g = exp(-exp(A_log)
// softplus(. + dt_bias)). tm_forget_gate_prepare: q <- silu(q), f <- low + (1 - low) sigmoid(f + bias).
// tm_talk_mix: out[t, h] = sum_g talk[h, g] o[t, g, value head of h].
#include "common.cuh"

namespace tmk {

constexpr int kGmThreads = 256;
constexpr int kGmChunk = 16;
constexpr int kGmRows = 16;
constexpr int kGmMaxTaps = 16;

struct GmGeometry {
  int parts, cols, d_pad;
};

inline GmGeometry gm_geometry(int d) {
  GmGeometry g;
  g.parts = 1;
  while (g.parts * kGmRows < d) g.parts *= 2;
  g.cols = kGmThreads / g.parts;
  g.d_pad = g.parts * kGmRows;
  return g;
}

__device__ __forceinline__ void gm_cp4(float* dst, const float* src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void gm_cp16(float* dst, const float* src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void gm_cp_wait() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// W consecutive elements per access (W = 4: 16 bytes of float, 8 of bfloat16; the pointer must be aligned so).
template <int W, typename T> __device__ __forceinline__ void ldw(const T* p, float (&v)[W]) {
  if constexpr (W == 4) load4(p, v);
  else v[0] = to_float(p[0]);
}
template <int W, typename T> __device__ __forceinline__ void stw(T* p, const float (&v)[W]) {
  if constexpr (W == 4) store4(p, v);
  else p[0] = from_float<T>(v[0]);
}

__device__ __forceinline__ float gm_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float gm_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// vec: bit 0 = the q and k columns, bit 1 = the v columns may be copied 16 bytes at a time.
template <int MODE, bool ROWDECAY, bool DELTA>
__global__ void __launch_bounds__(kGmThreads, 4) gated_memory_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int vec, const float* __restrict__ gb,
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* __restrict__ y, int heads, int qk_heads, int d, int dv, int parts, int cols,
    int slice_len, int max_slices, float* __restrict__ slice_S, int extra) {
  constexpr int R = kGmRows, chunk = kGmChunk;
  extern __shared__ __align__(16) float smem[];
  const int d_pad = parts * R;
  // one buffer: q [chunk][d_pad], k or f [chunk][d_pad], v [chunk][cols], g [chunk], beta [chunk]
  const int buf_floats = chunk * (2 * d_pad + cols) + 2 * chunk;

  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x, head = blockIdx.y;
  const int qk_head = head / (heads / qk_heads);
  const int s = MODE == 0 ? blockIdx.z : blockIdx.z / max_slices;
  const int sl = MODE == 0 ? 0 : blockIdx.z - s * max_slices;
  const int q_len = cu_q[s + 1] - cu_q[s];
  const int t_begin = MODE == 0 ? 0 : sl * slice_len;
  const int n_tok = (MODE == 0 ? q_len : min(q_len, t_begin + slice_len)) - t_begin;
  if (n_tok <= 0) return;
  const int first = cu_q[s] + t_begin;
  const int tid = threadIdx.x;
  const int part = tid % parts, col_local = tid / parts;
  const int col = tile * cols + col_local;
  const int n_cols = MODE == 1 ? dv + extra : dv;            // the first pass also walks the columns that record P
  const bool live = col < n_cols;
  const long long per = (long long)heads * (dv + extra) * d_pad;      // one slice's record in scratch
  float* record = MODE == 0 ? state + (size_t)state_slots[s] * state_stride + state_off
                            : slice_S + (size_t)blockIdx.z * per;
  const int rec_cols = MODE == 0 ? dv : dv + extra;
  float* S_g = record + ((size_t)head * rec_cols + (live ? col : 0)) * d_pad + part * 4;
  const int gs = 4 * parts;                                // rows between a lane's groups of four

  float S[R];
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    if (MODE == 1) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = (r >> 2) * gs + part * 4 + e;
        float v0 = 0.f;
        if (live && col >= dv && row < d) v0 = DELTA ? (row == col - dv ? 1.f : 0.f) : 1.f;
        S[r + e] = v0;
      }
    } else if (!live) {
      S[r] = S[r + 1] = S[r + 2] = S[r + 3] = 0.f;
    } else {
      const float4 x = *reinterpret_cast<const float4*>(S_g + (r >> 2) * gs);
      S[r] = x.x, S[r + 1] = x.y, S[r + 2] = x.z, S[r + 3] = x.w;
    }
  }
  // what the copies never write stays zero: rows >= d of q and k, columns >= dv of v
  for (int idx = tid; idx < 2 * buf_floats; idx += kGmThreads) smem[idx] = 0.f;
  __syncthreads();

  const int n_chunks = (n_tok + chunk - 1) / chunk;
  const int v_live = max(0, min(cols, dv - tile * cols));
  float row_live[ROWDECAY ? R : 1];                       // 1 for the rows that exist: the key 1 - f is 0 on the padding
  if (ROWDECAY) {
#pragma unroll
    for (int r = 0; r < R; ++r) row_live[r] = (r >> 2) * gs + part * 4 + (r & 3) < d ? 1.f : 0.f;
  }

  auto stage = [&](int ci) {                               // asynchronous copies of chunk ci into its buffer
    float* buf = smem + (ci & 1) * buf_floats;
    const int cn = min(chunk, n_tok - ci * chunk);
    const float* base = proj + (size_t)(first + ci * chunk) * ld;
    if (vec & 1) {
      const int d4 = d >> 2;
      for (int idx = tid; idx < cn * d4; idx += kGmThreads) {
        const int tt = idx / d4, e = (idx - tt * d4) << 2;
        const float* row = base + (size_t)tt * ld;
        if (MODE != 1) gm_cp16(buf + tt * d_pad + e, row + q_col + qk_head * d + e);
        gm_cp16(buf + (chunk + tt) * d_pad + e, row + k_col + qk_head * d + e);
      }
    } else {
      for (int idx = tid; idx < cn * d; idx += kGmThreads) {
        const int tt = idx / d, e = idx - tt * d;
        const float* row = base + (size_t)tt * ld;
        if (MODE != 1) gm_cp4(buf + tt * d_pad + e, row + q_col + qk_head * d + e);
        gm_cp4(buf + (chunk + tt) * d_pad + e, row + k_col + qk_head * d + e);
      }
    }
    float* vb = buf + 2 * chunk * d_pad;
    const float* vsrc = base + v_col + head * dv + tile * cols;
    if (vec & 2) {
      const int v4 = v_live >> 2;
      for (int idx = tid; idx < cn * v4; idx += kGmThreads) {
        const int tt = idx / v4, cc = (idx - tt * v4) << 2;
        gm_cp16(vb + tt * cols + cc, vsrc + (size_t)tt * ld + cc);
      }
    } else {
      for (int idx = tid; idx < cn * v_live; idx += kGmThreads) {
        const int tt = idx / v_live, cc = idx - tt * v_live;
        gm_cp4(vb + tt * cols + cc, vsrc + (size_t)tt * ld + cc);
      }
    }
    if (!ROWDECAY || DELTA) {
      float* gbuf = buf + chunk * (2 * d_pad + cols);
      if (tid < 2 * cn) {
        const int tt = tid >> 1, which = tid & 1;
        gm_cp4(gbuf + which * chunk + tt, gb + (size_t)(first + ci * chunk + tt) * 2 * heads + which * heads + head);
      }
    }
  };

  stage(0);
  gm_cp_wait();
  __syncthreads();
  for (int ci = 0; ci < n_chunks; ++ci) {
    const bool more = ci + 1 < n_chunks;
    if (more) stage(ci + 1);
    const float* buf = smem + (ci & 1) * buf_floats;
    const float* qs = buf + part * 4;
    const float* ks = buf + chunk * d_pad + part * 4;
    const float* vs = buf + 2 * chunk * d_pad + col_local;
    const float* gsm = buf + chunk * (2 * d_pad + cols);
    const int cn = min(chunk, n_tok - ci * chunk);
    float* y_row = y + (size_t)(first + ci * chunk) * heads * dv + (size_t)head * dv + (live && col < dv ? col : 0);
#pragma unroll 2
    for (int tt = 0; tt < cn; ++tt) {
      const float v = vs[tt * cols];
      const float* kr = ks + tt * d_pad;
      const float* qr = qs + tt * d_pad;
      float k_reg[R];
      if (ROWDECAY) {
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 f4 = *reinterpret_cast<const float4*>(kr + (r >> 2) * gs);
          // S <- f S + (1 - f) v = v + f (S - v) on the rows that exist; rows >= d read f = 0 and stay 0
          S[r] = fmaf(f4.x, S[r] - v, v * row_live[r]);
          S[r + 1] = fmaf(f4.y, S[r + 1] - v, v * row_live[r + 1]);
          S[r + 2] = fmaf(f4.z, S[r + 2] - v, v * row_live[r + 2]);
          S[r + 3] = fmaf(f4.w, S[r + 3] - v, v * row_live[r + 3]);
        }
      } else {
        const float g = gsm[tt];
        float c0 = 0.f, c1 = 0.f;
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + (r >> 2) * gs);
          k_reg[r] = k4.x, k_reg[r + 1] = k4.y, k_reg[r + 2] = k4.z, k_reg[r + 3] = k4.w;
          if (DELTA) {            // the sum down the column runs on the memory before its decay; g enters afterwards
            c0 = fmaf(S[r], k4.x, c0);
            c1 = fmaf(S[r + 1], k4.y, c1);
            c0 = fmaf(S[r + 2], k4.z, c0);
            c1 = fmaf(S[r + 3], k4.w, c1);
          } else {
            S[r] = fmaf(g, S[r], k4.x * v);
            S[r + 1] = fmaf(g, S[r + 1], k4.y * v);
            S[r + 2] = fmaf(g, S[r + 2], k4.z * v);
            S[r + 3] = fmaf(g, S[r + 3], k4.w * v);
          }
        }
        if (DELTA) {
          float c = c0 + c1;
          for (int off = parts >> 1; off > 0; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
          const float u = gsm[chunk + tt] * (v - g * c);
#pragma unroll
          for (int r = 0; r < R; ++r) S[r] = fmaf(g, S[r], k_reg[r] * u);
        }
      }
      if (MODE != 1) {
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + (r >> 2) * gs);
          o0 = fmaf(S[r], q4.x, o0);
          o1 = fmaf(S[r + 1], q4.y, o1);
          o0 = fmaf(S[r + 2], q4.z, o0);
          o1 = fmaf(S[r + 3], q4.w, o1);
        }
        float o = o0 + o1;
        for (int off = parts >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
        if (part == 0 && live) y_row[(size_t)tt * heads * dv] = o;
      }
    }
    gm_cp_wait();
    __syncthreads();
  }
  if (MODE != 2 && live) {
#pragma unroll
    for (int r = 0; r < R; r += 4)
      *reinterpret_cast<float4*>(S_g + (r >> 2) * gs) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
  }
}

// Between the two passes over time slices. One block per (tile of CT columns, head, request): slice k's own memory in
// scratch becomes the memory at its start, S <- P S + own from slice to slice, and the slot receives the memory after
// the last slice. Diagonal P: one number per row (column dv of the record). Full P (delta rule): column dv + j of the
// record holds P[:, j]; the tile's columns of S go through shared memory so that every row reads them all. Thread
// (row r, share js): the sum over j is dealt out over JS threads a row, which meet in shared memory in the order of js.
constexpr int kGmPassCols = 8;

static_assert(kGmPassCols == 8, "a row of the tile is two 16-byte loads");
// acc[c] += p * row[c] for the tile's eight columns; row lies in shared memory, 32-byte aligned.
__device__ __forceinline__ void row_fma(float (&acc)[kGmPassCols], float p, const float* row) {
  const float4 a = *reinterpret_cast<const float4*>(row), b = *reinterpret_cast<const float4*>(row + 4);
  acc[0] = fmaf(p, a.x, acc[0]), acc[1] = fmaf(p, a.y, acc[1]), acc[2] = fmaf(p, a.z, acc[2]), acc[3] = fmaf(p, a.w, acc[3]);
  acc[4] = fmaf(p, b.x, acc[4]), acc[5] = fmaf(p, b.y, acc[5]), acc[6] = fmaf(p, b.z, acc[6]), acc[7] = fmaf(p, b.w, acc[7]);
}

// JP: a thread's share of the sum over j when every share has exactly that many numbers (d = JS * JP: no tests inside the
// loops, the share's rows of P wholly prefetched); 0: any shape.
template <bool DELTA, int JP>
__global__ void __launch_bounds__(512) gated_memory_pass_states_kernel(
    float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, float* slice_S, int heads, int d, int dv, int d_pad, int slice_len, int max_slices,
    int extra, int JS) {
  extern __shared__ __align__(16) float pass_s[];          // cur [d_pad][CT] (a row's CT numbers side by side), then partial sums [JS][CT][d_pad]
  float* cur_s = pass_s;
  float* part_s = pass_s + kGmPassCols * d_pad;
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.y, s = blockIdx.z, r = threadIdx.x % d_pad, js = threadIdx.x / d_pad;
  const int q_len = cu_q[s + 1] - cu_q[s];
  if (q_len <= 0) return;
  const int c0 = blockIdx.x * kGmPassCols;
  const int nc = min(kGmPassCols, dv - c0);
  const int slices = (q_len + slice_len - 1) / slice_len;
  const long long per = (long long)heads * (dv + extra) * d_pad;
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off + ((size_t)head * dv + c0) * d_pad + r;
  float cur[kGmPassCols];
#pragma unroll
  for (int c = 0; c < kGmPassCols; ++c) cur[c] = (c < nc && js == 0) ? slot[(size_t)c * d_pad] : 0.f;
  const int j_per = (d + JS - 1) / JS;
  const int j_lo = js * j_per, j_hi = min(d, j_lo + j_per);
  // P does not depend on the chain: a slice's first kPre numbers of this thread's share of P[r, :] are loaded while the
  // slice before it is multiplied, so that the chain waits for arithmetic only (shares of up to kPre numbers wholly).
  constexpr int kPre = JP ? JP : 32;
  float p_next[kPre];
  auto prefetch = [&](int k) {
    const float* P = slice_S + ((size_t)s * max_slices + k) * per + ((size_t)head * (dv + extra) + dv + j_lo) * d_pad + r;
#pragma unroll
    for (int u = 0; u < kPre; ++u) {
      if (JP || j_lo + u < j_hi) p_next[u] = *P;
      else p_next[u] = 0.f;
      P += d_pad;
    }
  };
  if (DELTA) prefetch(0);
  for (int k = 0; k < slices; ++k) {
    float* rec = slice_S + ((size_t)s * max_slices + k) * per + (size_t)head * (dv + extra) * d_pad;
    float* mine = rec + (size_t)c0 * d_pad + r;
    float own[kGmPassCols];
#pragma unroll
    for (int c = 0; c < kGmPassCols; ++c) own[c] = (c < nc && js == 0) ? mine[(size_t)c * d_pad] : 0.f;
    if (DELTA) {
      float p_cur[kPre];
#pragma unroll
      for (int u = 0; u < kPre; ++u) p_cur[u] = p_next[u];
      if (k + 1 < slices) prefetch(k + 1);
      __syncthreads();
      if (js == 0) {
        *reinterpret_cast<float4*>(cur_s + r * kGmPassCols) = make_float4(cur[0], cur[1], cur[2], cur[3]);
        *reinterpret_cast<float4*>(cur_s + r * kGmPassCols + 4) = make_float4(cur[4], cur[5], cur[6], cur[7]);
      }
      __syncthreads();
      const float* P = rec + (size_t)dv * d_pad + r;         // P[r, j] at P[j * d_pad]
      float acc[kGmPassCols];
#pragma unroll
      for (int c = 0; c < kGmPassCols; ++c) acc[c] = 0.f;
      const float* rows = cur_s + j_lo * kGmPassCols;
#pragma unroll
      for (int u = 0; u < kPre; ++u) {
        if (JP || j_lo + u < j_hi) row_fma(acc, p_cur[u], rows + u * kGmPassCols);
      }
      int j = JP ? j_hi : j_lo + kPre;
      for (; j + 8 <= j_hi; j += 8) {                        // the rest of a long share: eight loads in flight
        float p[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) p[u] = P[(size_t)(j + u) * d_pad];
#pragma unroll
        for (int u = 0; u < 8; ++u) row_fma(acc, p[u], cur_s + (j + u) * kGmPassCols);
      }
      for (; j < j_hi; ++j) {
        row_fma(acc, P[(size_t)j * d_pad], cur_s + j * kGmPassCols);
      }
      if (JS > 1) {
#pragma unroll
        for (int c = 0; c < kGmPassCols; ++c) part_s[(js * kGmPassCols + c) * d_pad + r] = acc[c];
        __syncthreads();
        if (js == 0) {
          for (int o = 0; o < JS; ++o)
#pragma unroll
            for (int c = 0; c < kGmPassCols; ++c) own[c] += part_s[(o * kGmPassCols + c) * d_pad + r];
        }
      } else {
#pragma unroll
        for (int c = 0; c < kGmPassCols; ++c) own[c] += acc[c];
      }
    } else {
      const float f = rec[(size_t)dv * d_pad + r];
#pragma unroll
      for (int c = 0; c < kGmPassCols; ++c) own[c] = fmaf(f, cur[c], own[c]);
    }
    if (js == 0) {
#pragma unroll
      for (int c = 0; c < kGmPassCols; ++c) {
        if (c < nc) mine[(size_t)c * d_pad] = cur[c];
        cur[c] = own[c];
      }
    }
  }
  if (js == 0) {
#pragma unroll
    for (int c = 0; c < kGmPassCols; ++c)
      if (c < nc) slot[(size_t)c * d_pad] = cur[c];
  }
}

// Thread (token, VEC channels). Only the thread of a request's first row touches the slot: it computes the up to
// taps - 1 outputs that need carried inputs, then writes the step's last taps - 1 inputs back. TAPS: the number of taps
// when it is 1 to 5 (loops unrolled, everything in registers), 0 for any number up to kGmMaxTaps.
template <int VEC, int TAPS>
__global__ void __launch_bounds__(128) short_conv_state_kernel(
    const float* __restrict__ proj, long long ld, int col0, int channels, int taps_rt, const float* __restrict__ weight,
    const float* __restrict__ bias, float* __restrict__ state, long long state_stride, long long state_off,
    const int* __restrict__ cu_q, const int* __restrict__ seq_of_token, const int* __restrict__ state_slots, int act,
    float* __restrict__ out, long long out_ld, int out_col0) {
  constexpr int NT = TAPS ? TAPS : kGmMaxTaps;
  const int taps = TAPS ? TAPS : taps_rt;
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (c0 >= channels) {
    pdl_wait();
    return;
  }
  float w[VEC][NT], bv[VEC];                 // (weights: before the wait)
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    bv[e] = bias ? bias[c0 + e] : 0.f;
#pragma unroll
    for (int k = 0; k < NT; ++k) w[e][k] = k < taps ? weight[(size_t)(c0 + e) * taps + k] : 0.f;
  }
  pdl_wait();
  const int s = seq_of_token[t];
  const int first = cu_q[s];
  const int j = t - first;
  const int carried = taps - 1;
  if (j > 0 && j < carried) return;          // the first row's thread computes these
  auto load = [&](int row, float (&u)[VEC]) {
    const float* src = proj + (size_t)row * ld + col0 + c0;
    if constexpr (VEC == 4) {
      const float4 x = *reinterpret_cast<const float4*>(src);
      u[0] = x.x + bv[0], u[1] = x.y + bv[1], u[2] = x.z + bv[2], u[3] = x.w + bv[3];
    } else {
      u[0] = src[0] + bv[0];
    }
  };
  auto store = [&](int row, const float (&acc)[VEC]) {
    float* dst = out + (size_t)row * out_ld + out_col0 + c0;
#pragma unroll
    for (int e = 0; e < VEC; ++e) dst[e] = act ? acc[e] / (1.0f + expf(-acc[e])) : acc[e];
  };
  if (j >= carried) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
    for (int k = 0; k < NT; ++k) {
      if (k >= taps) break;
      float u[VEC];
      load(t - carried + k, u);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(w[e][k], u[e], acc[e]);
    }
    store(t, acc);
    return;
  }
  // j == 0: this thread owns the request's carried inputs of its channels. win[i] for i < carried: the inputs before
  // the step, oldest first; from there on the step's own rows.
  const int q_len = cu_q[s + 1] - first;
  float* slot = state + (size_t)state_slots[s] * state_stride + state_off + c0;     // carried input i at slot[i * channels]
  float win[2 * NT][VEC];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    if (i >= carried) break;
#pragma unroll
    for (int e = 0; e < VEC; ++e) win[i][e] = slot[(size_t)i * channels + e];
  }
  const int n_head = min(max(carried, 1), q_len);        // rows this thread computes (one tap: the row itself)
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    if (i >= n_head) break;
    load(first + i, win[NT == kGmMaxTaps ? carried + i : TAPS - 1 + i]);
  }
#pragma unroll
  for (int jj = 0; jj < NT; ++jj) {
    if (jj >= n_head) break;
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
    for (int k = 0; k < NT; ++k) {
      if (k >= taps) break;
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(w[e][k], win[jj + k][e], acc[e]);
    }
    store(first + jj, acc);
  }
  // the step's last `carried` inputs: row q_len - carried + i of the step, or what was carried when the step is shorter
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    if (i >= carried) break;
    const int src = q_len - carried + i;
    float u[VEC];
    if (src >= n_head) {
      load(first + src, u);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) u[e] = 0.f;
#pragma unroll
      for (int m = 0; m < 2 * NT; ++m)                   // win[carried + src], picked without indexing the registers
        if (m == carried + src) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[e] = win[m][e];
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) slot[(size_t)i * channels + e] = u[e];
  }
}

// One block per token. x [T, x_ld]: q at q_col and k at k_col (qk_heads x d), changed in place. raw [T, raw_ld]: the
// projections of beta (b_col) and of the decay (a_col), heads numbers each. gb [T, 2 heads] <- (g, beta).
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* __restrict__ x, long long x_ld, int q_col, int k_col,
                                                            int qk_heads, int d, float q_scale, float unit_eps,
                                                            const float* __restrict__ raw, long long raw_ld, int b_col,
                                                            int a_col, const float* __restrict__ A_log,
                                                            const float* __restrict__ dt_bias, int heads,
                                                            float* __restrict__ gb) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  float* row = x + (size_t)t * x_ld;
  for (int u = warp; u < 2 * qk_heads; u += n_warps) {      // units: the q heads, then the k heads
    const bool is_q = u < qk_heads;
    float* hp = row + (is_q ? q_col + u * d : k_col + (u - qk_heads) * d);
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(hp[i], hp[i], ss);
    const float f = (is_q ? q_scale : 1.0f) / sqrtf(warp_sum(ss) + unit_eps);
    for (int i = lane; i < d; i += 32) hp[i] *= f;
  }
  const float* r = raw + (size_t)t * raw_ld;
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    gb[(size_t)t * 2 * heads + h] = expf(-expf(A_log[h]) * gm_softplus(r[a_col + h] + dt_bias[h]));
    gb[(size_t)t * 2 * heads + heads + h] = gm_sigmoid(r[b_col + h]);
  }
}

// x [T, ld]: q at q_col <- silu(q); f at f_col <- low + (1 - low) sigmoid(f + bias); n numbers each.
__global__ void __launch_bounds__(256) forget_gate_prepare_kernel(float* __restrict__ x, long long ld, int q_col, int f_col,
                                                                  int n, const float* __restrict__ low,
                                                                  const float* __restrict__ bias) {
  pdl_launch_dependents();
  pdl_wait();
  float* row = x + (size_t)blockIdx.y * ld;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float q = row[q_col + i];
    row[q_col + i] = q / (1.0f + expf(-q));
    const float lo = low[i];
    row[f_col + i] = lo + (1.0f - lo) * gm_sigmoid(row[f_col + i] + (bias ? bias[i] : 0.f));
  }
}

// o [T, H, G, dv] float: head g's softmax weights applied to the values of every key/value head. out[t, h, :] =
// scale * sum_g talk[h, g] o[t, g, h / (H / G), :]. One block per token, a thread per four neighbouring numbers of the
// output where dv allows; talk lies in shared memory and four heads' loads are in flight at a time.
template <typename T, int W>
__global__ void __launch_bounds__(256) talk_mix_kernel(const float* __restrict__ o, const float* __restrict__ talk,
                                                       T* __restrict__ out, int H, int G, int dv, float scale,
                                                       long long out_ld) {
  extern __shared__ float talk_s[];
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) talk_s[i] = talk[i];      // (weights: before the wait)
  pdl_wait();
  __syncthreads();
  const size_t t = blockIdx.x;
  const int Gq = H / G;
  for (int idx = threadIdx.x * W; idx < H * dv; idx += blockDim.x * W) {
    const int h = idx / dv, e = idx - h * dv;
    const int c = h / Gq;
    const float* src = o + ((t * H) * G + c) * dv + e;       // head g's at src + g * G * dv
    const float* tw = talk_s + h * H;
    float acc[W];
#pragma unroll
    for (int i = 0; i < W; ++i) acc[i] = 0.f;
    int g = 0;
    for (; g + 4 <= H; g += 4) {
      float x[4][W];
#pragma unroll
      for (int u = 0; u < 4; ++u) ldw<W>(src + (size_t)(g + u) * G * dv, x[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < W; ++i) acc[i] = fmaf(tw[g + u], x[u][i], acc[i]);
    }
    for (; g < H; ++g) {
      float x[W];
      ldw<W>(src + (size_t)g * G * dv, x);
#pragma unroll
      for (int i = 0; i < W; ++i) acc[i] = fmaf(tw[g], x[i], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < W; ++i) acc[i] *= scale;
    stw<W>(out + t * out_ld + idx, acc);
  }
}

}  // namespace tmk

using namespace tmk;

// proj: float, token t's row at proj + t * ld, q at q_col and k (row decays: f) at k_col (qk_heads x d), v at v_col
// (heads x dv); gb [T, 2 heads] float (g, beta) or null with row decays; a request's memories ([heads][dv][d_pad]
// floats) start state_off floats into its slot of `state` (state_off and state_stride multiples of 4); y [T, heads * dv]
// float. row_decay / delta pick the rule. mode 0: one walk per request. modes 1 and 2: the first and third pass over
// time slices of slice_len tokens, max_slices per request, through slice_S [n_seqs * max_slices] records of
// heads * (dv + extra) * d_pad floats, extra = d with the delta rule, else 1, with tm_gated_memory_pass_states between.
extern "C" int tm_gated_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, const float* gb, int row_decay,
                               int delta, float* state, long long state_stride, long long state_off, const int* cu_q,
                               const int* state_slots, float* y, int n_seqs, int heads, int qk_heads, int d, int dv, int mode,
                               int slice_len, int max_slices, float* slice_S, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || qk_heads < 1 || heads % qk_heads || d < 1 || d > 512 || dv < 1 || mode < 0 || mode > 2 ||
      (state_stride & 3) || (state_off & 3) || ((uintptr_t)state & 15) || (row_decay && delta) || (!(row_decay && !delta) && !gb))
    return TM_ERR_UNSUPPORTED_SHAPE;
  if (mode != 0 && (slice_len < 1 || max_slices < 1 || !slice_S || ((uintptr_t)slice_S & 15))) return TM_ERR_SCRATCH_TOO_SMALL;
  const GmGeometry g = gm_geometry(d);
  const int extra = delta ? d : 1;
  const bool rows16 = !((uintptr_t)proj & 15) && !(ld & 3);
  const int vec = (rows16 && !(q_col & 3) && !(k_col & 3) && !(d & 3) ? 1 : 0) | (rows16 && !(v_col & 3) && !(dv & 3) ? 2 : 0);
  const size_t smem = sizeof(float) * 2 * (kGmChunk * (2 * (size_t)g.d_pad + g.cols) + 2 * kGmChunk);
  const int n_cols = mode == 1 ? dv + extra : dv;
  const dim3 grid((n_cols + g.cols - 1) / g.cols, heads, n_seqs * (mode == 0 ? 1 : max_slices));
#define TM_GM_LAUNCH(M_, RD_, DL_)                                                                                         \
  {                                                                                                                        \
    auto kern = gated_memory_kernel<M_, RD_, DL_>;                                                                         \
    if (smem > 48 * 1024) {                                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
      if (e != cudaSuccess) return (int)e;                                                                                 \
    }                                                                                                                      \
    return launch_pdl(kern, grid, dim3(kGmThreads), smem, stream, proj, ld, q_col, k_col, v_col, vec, gb, state, state_stride, \
                      state_off, cu_q, state_slots, y, heads, qk_heads, d, dv, g.parts, g.cols, slice_len, max_slices,     \
                      slice_S, extra);                                                                                     \
  }
#define TM_GM_RULE(M_)                                   \
  if (row_decay) TM_GM_LAUNCH(M_, true, false)           \
  if (delta) TM_GM_LAUNCH(M_, false, true)               \
  TM_GM_LAUNCH(M_, false, false)
  if (mode == 0) { TM_GM_RULE(0) }
  if (mode == 1) { TM_GM_RULE(1) }
  TM_GM_RULE(2)
#undef TM_GM_RULE
#undef TM_GM_LAUNCH
}

extern "C" int tm_gated_memory_pass_states(float* state, long long state_stride, long long state_off, const int* cu_q,
                                           const int* state_slots, float* slice_S, int delta, int n_seqs, int heads, int d,
                                           int dv, int slice_len, int max_slices, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || d < 1 || d > 512 || dv < 1 || slice_len < 1 || max_slices < 1 || !slice_S || (state_stride & 3) ||
      (state_off & 3))
    return TM_ERR_UNSUPPORTED_SHAPE;
  const GmGeometry g = gm_geometry(d);
  const dim3 grid((dv + kGmPassCols - 1) / kGmPassCols, heads, n_seqs);
  if (delta) {
    const int JS = 512 / g.d_pad;         // threads that share a row's sum over j (1 for memories of 512 rows)
    const size_t smem = sizeof(float) * kGmPassCols * g.d_pad * (1 + (JS > 1 ? JS : 0));
#define TM_GM_CHAIN(JP_)                                                                                                   \
  {                                                                                                                        \
    auto kern = gated_memory_pass_states_kernel<true, JP_>;                                                                \
    if (smem > 48 * 1024) {                                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
      if (e != cudaSuccess) return (int)e;                                                                                 \
    }                                                                                                                      \
    return launch_pdl(kern, grid, dim3(g.d_pad * JS), smem, stream, state, state_stride, state_off, cu_q, state_slots,     \
                      slice_S, heads, d, dv, g.d_pad, slice_len, max_slices, d, JS);                                       \
  }
    if (d == JS * 32) TM_GM_CHAIN(32)
    if (d == JS * 8) TM_GM_CHAIN(8)
    TM_GM_CHAIN(0)
#undef TM_GM_CHAIN
  }
  return launch_pdl(gated_memory_pass_states_kernel<false, 0>, grid, dim3(g.d_pad), 0, stream, state, state_stride, state_off,
                    cu_q, state_slots, slice_S, heads, d, dv, g.d_pad, slice_len, max_slices, 1, 1);
}

// proj: float, element (t, c) of the input at proj + t * ld + col0 + c; weight [channels, taps] float (the last tap weighs
// the current token); bias [channels] float or null, added to the input before the convolution (the carried inputs hold
// it); a request's carried inputs [taps - 1, channels] start state_off floats into its slot; act 0: none, 1: silu; out:
// float, element (t, c) at out + t * out_ld + out_col0 + c. out must not alias proj.
extern "C" int tm_short_conv_state(const float* proj, long long ld, int col0, int channels, int taps, const float* weight,
                                   const float* bias, float* state, long long state_stride, long long state_off,
                                   const int* cu_q, const int* seq_of_token, const int* state_slots, int act, float* out,
                                   long long out_ld, int out_col0, int T_rows, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (taps < 1 || taps > kGmMaxTaps || channels < 1 || (act != 0 && act != 1)) return TM_ERR_UNSUPPORTED_SHAPE;
  const bool wide = !(channels & 3) && !(col0 & 3) && !(ld & 3) && !((uintptr_t)proj & 15);
#define TM_CONV(VEC_, TAPS_)                                                                                                \
  return launch_pdl(short_conv_state_kernel<VEC_, TAPS_>, dim3(T_rows, (channels / VEC_ + 127) / 128), dim3(128), 0, stream, \
                    proj, ld, col0, channels, taps, weight, bias, state, state_stride, state_off, cu_q, seq_of_token,       \
                    state_slots, act, out, out_ld, out_col0)
  if (wide) {
    switch (taps) {
      case 1: TM_CONV(4, 1);
      case 2: TM_CONV(4, 2);
      case 3: TM_CONV(4, 3);
      case 4: TM_CONV(4, 4);
      case 5: TM_CONV(4, 5);
      default: break;
    }
  }
  switch (taps) {
    case 1: TM_CONV(1, 1);
    case 2: TM_CONV(1, 2);
    case 3: TM_CONV(1, 3);
    case 4: TM_CONV(1, 4);
    case 5: TM_CONV(1, 5);
    default: TM_CONV(1, 0);
  }
#undef TM_CONV
}

extern "C" int tm_delta_prepare(float* x, long long x_ld, int q_col, int k_col, int qk_heads, int d, float q_scale,
                                float unit_eps, const float* raw, long long raw_ld, int b_col, int a_col, const float* A_log,
                                const float* dt_bias, int heads, float* gb, int T_rows, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (qk_heads < 1 || heads < 1 || d < 1) return TM_ERR_UNSUPPORTED_SHAPE;
  return launch_pdl(delta_prepare_kernel, dim3(T_rows), dim3(128), 0, stream, x, x_ld, q_col, k_col, qk_heads, d, q_scale,
                    unit_eps, raw, raw_ld, b_col, a_col, A_log, dt_bias, heads, gb);
}

extern "C" int tm_forget_gate_prepare(float* x, long long ld, int q_col, int f_col, int n, const float* low, const float* bias,
                                      int T_rows, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (n < 1) return TM_ERR_UNSUPPORTED_SHAPE;
  return launch_pdl(forget_gate_prepare_kernel, dim3((unsigned)std::min(16, (n + 255) / 256), T_rows), dim3(256), 0, stream, x,
                    ld, q_col, f_col, n, low, bias);
}

// out: element (t, c) at out + t * out_ld + c, c < H dv (the heads may be columns of a wider matrix).
extern "C" int tm_talk_mix(int dtype, const float* o, const float* talk, void* out, long long out_ld, float scale, int T_rows,
                           int H, int G, int dv, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (H < 1 || G < 1 || H % G || dv < 1 || H > 96) return TM_ERR_UNSUPPORTED_SHAPE;
  const size_t smem = sizeof(float) * H * H;
  const bool wide = !(dv & 3) && !(out_ld & 3) && !(((uintptr_t)o | (uintptr_t)out) & 15);
#define TM_TALK(T_, W_)                                                                                              \
  return launch_pdl(talk_mix_kernel<T_, W_>, dim3(T_rows), dim3(256), smem, stream, o, talk, (T_*)out, H, G, dv, scale, out_ld)
  if (dtype == TM_DTYPE_F32) {
    if (wide) TM_TALK(float, 4);
    TM_TALK(float, 1);
  }
  if (dtype == TM_DTYPE_BF16) {
    if (wide) TM_TALK(__nv_bfloat16, 4);
    TM_TALK(__nv_bfloat16, 1);
  }
#undef TM_TALK
  return TM_ERR_BAD_DTYPE;
}
