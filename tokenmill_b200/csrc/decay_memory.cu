// Linear attention with a constant decay per head: per head a d x dv memory S, from the state the request's slot holds,
//   S_t = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t
// with q, k (heads x d) and v (heads x dv) column ranges of one 32-bit projection, each passed through an activation on
// the way in (0: none, 1: silu). The memory, the products and the sums are 32-bit in both run dtypes; o is written in
// 32-bit for the norm that follows.
//
// One block of 256 threads per (tile of columns, head, request or time slice). A column's d numbers are spread over
// `parts` neighbouring lanes, 16 rows each in registers (parts = the power of two >= d / 16; lane p takes rows
// 4 p .. 4 p + 3 of every group of 4 * parts rows, so that neighbouring lanes read neighbouring 16 bytes of k and q in
// shared memory and of S in the slot), and the product with q is finished by shuffles among those lanes. A request's
// memories are laid out [heads][dv][d_pad], a column's rows side by side (d_pad = 16 * parts; rows >= d stay zero).
// Tokens pass through shared memory sixteen at a time in two buffers: while the block walks one buffer strictly in
// order, the next sixteen tokens' q, k and v columns arrive by asynchronous copies (16 bytes each where the columns
// are aligned so). With an activation the block applies it to a buffer once it has arrived; tm_decay_activate applies
// it to the projection's columns in place instead, once for all blocks, which is what long portions use.
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

constexpr int kDecayThreads = 256;
constexpr int kDecayChunk = 16;
constexpr int kDecayRows = 16;

struct DecayGeometry {
  int parts, cols, col_tiles, d_pad;
  long long floats;
};

inline DecayGeometry decay_geometry(int heads, int d, int dv) {
  DecayGeometry g;
  g.parts = 1;
  while (g.parts * kDecayRows < d) g.parts *= 2;
  g.cols = kDecayThreads / g.parts;
  g.col_tiles = (dv + g.cols - 1) / g.cols;
  g.d_pad = g.parts * kDecayRows;
  g.floats = (long long)heads * dv * g.d_pad;
  return g;
}

__device__ __forceinline__ float act_in(float v, int act) { return act == 1 ? v / (1.0f + expf(-v)) : v; }

__device__ __forceinline__ void decay_cp4(float* dst, const float* src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void decay_cp16(float* dst, const float* src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void decay_cp_wait() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// vec: bit 0 = the q and k columns, bit 1 = the v columns may be copied 16 bytes at a time.
template <int MODE>
__global__ void __launch_bounds__(kDecayThreads, 4) decay_memory_kernel(
    const float* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, int act, int vec,
    const float* __restrict__ decay, float* __restrict__ state, long long state_stride, long long state_off,
    const int* __restrict__ cu_q, const int* __restrict__ state_slots, float* __restrict__ y, int heads, int d, int dv,
    int parts, int cols, int slice_len, int max_slices, float* __restrict__ slice_S) {
  constexpr int R = kDecayRows, chunk = kDecayChunk;
  extern __shared__ __align__(16) float smem[];
  const int d_pad = parts * R;
  const int buf_floats = chunk * (2 * d_pad + cols);       // one buffer: q [chunk][d_pad], k [chunk][d_pad], v [chunk][cols]

  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x, head = blockIdx.y;
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
  const bool live = col < dv;
  const long long per = (long long)heads * dv * d_pad;
  float* record = MODE == 0 ? state + (size_t)state_slots[s] * state_stride + state_off : slice_S + (size_t)blockIdx.z * per;
  float* S_g = record + ((size_t)head * dv + (live ? col : 0)) * d_pad + part * 4;
  const int gs = 4 * parts;                                // rows between a lane's groups of four
  const float a = decay[head];

  float S[R];
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    if (MODE == 1 || !live) {
      S[r] = S[r + 1] = S[r + 2] = S[r + 3] = 0.f;
    } else {
      const float4 x = *reinterpret_cast<const float4*>(S_g + (r >> 2) * gs);
      S[r] = x.x, S[r + 1] = x.y, S[r + 2] = x.z, S[r + 3] = x.w;
    }
  }
  // what the copies never write stays zero: rows >= d of q and k, columns >= dv of v
  for (int idx = tid; idx < 2 * buf_floats; idx += kDecayThreads) smem[idx] = 0.f;
  __syncthreads();

  const int n_chunks = (n_tok + chunk - 1) / chunk;
  const int v_live = max(0, min(cols, dv - tile * cols));

  auto stage = [&](int ci) {                               // asynchronous copies of chunk ci into its buffer
    float* buf = smem + (ci & 1) * buf_floats;
    const int cn = min(chunk, n_tok - ci * chunk);
    const float* base = proj + (size_t)(first + ci * chunk) * ld;
    if (vec & 1) {
      const int d4 = d >> 2;
      for (int idx = tid; idx < cn * d4; idx += kDecayThreads) {
        const int tt = idx / d4, e = (idx - tt * d4) << 2;
        const float* row = base + (size_t)tt * ld;
        if (MODE != 1) decay_cp16(buf + tt * d_pad + e, row + q_col + head * d + e);
        decay_cp16(buf + (chunk + tt) * d_pad + e, row + k_col + head * d + e);
      }
    } else {
      for (int idx = tid; idx < cn * d; idx += kDecayThreads) {
        const int tt = idx / d, e = idx - tt * d;
        const float* row = base + (size_t)tt * ld;
        if (MODE != 1) decay_cp4(buf + tt * d_pad + e, row + q_col + head * d + e);
        decay_cp4(buf + (chunk + tt) * d_pad + e, row + k_col + head * d + e);
      }
    }
    float* vb = buf + 2 * chunk * d_pad;
    const float* vsrc = base + v_col + head * dv + tile * cols;
    if (vec & 2) {
      const int v4 = v_live >> 2;
      for (int idx = tid; idx < cn * v4; idx += kDecayThreads) {
        const int tt = idx / v4, cc = (idx - tt * v4) << 2;
        decay_cp16(vb + tt * cols + cc, vsrc + (size_t)tt * ld + cc);
      }
    } else {
      for (int idx = tid; idx < cn * v_live; idx += kDecayThreads) {
        const int tt = idx / v_live, cc = idx - tt * v_live;
        decay_cp4(vb + tt * cols + cc, vsrc + (size_t)tt * ld + cc);
      }
    }
  };
  auto activate = [&](int ci) {                            // act(0) = 0, so the padding may pass through it too
    float* buf = smem + (ci & 1) * buf_floats;
    for (int idx = tid; idx < buf_floats; idx += kDecayThreads) buf[idx] = act_in(buf[idx], act);
  };

  stage(0);
  decay_cp_wait();
  __syncthreads();
  if (act) {
    activate(0);
    __syncthreads();
  }
  for (int ci = 0; ci < n_chunks; ++ci) {
    const bool more = ci + 1 < n_chunks;
    if (more) stage(ci + 1);
    const float* buf = smem + (ci & 1) * buf_floats;
    const float* qs = buf + part * 4;
    const float* ks = buf + chunk * d_pad + part * 4;
    const float* vs = buf + 2 * chunk * d_pad + col_local;
    const int cn = min(chunk, n_tok - ci * chunk);
    float* y_row = y + (size_t)(first + ci * chunk) * heads * dv + (size_t)head * dv + (live ? col : 0);
#pragma unroll 2
    for (int tt = 0; tt < cn; ++tt) {
      const float v = vs[tt * cols];
      const float* kr = ks + tt * d_pad;
      const float* qr = qs + tt * d_pad;
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kr + (r >> 2) * gs);
        S[r] = fmaf(a, S[r], k4.x * v);
        S[r + 1] = fmaf(a, S[r + 1], k4.y * v);
        S[r + 2] = fmaf(a, S[r + 2], k4.z * v);
        S[r + 3] = fmaf(a, S[r + 3], k4.w * v);
        if (MODE != 1) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + (r >> 2) * gs);
          o0 = fmaf(S[r], q4.x, o0);
          o1 = fmaf(S[r + 1], q4.y, o1);
          o0 = fmaf(S[r + 2], q4.z, o0);
          o1 = fmaf(S[r + 3], q4.w, o1);
        }
      }
      if (MODE != 1) {
        float o = o0 + o1;
        for (int off = parts >> 1; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
        if (part == 0 && live) y_row[(size_t)tt * heads * dv] = o;
      }
    }
    decay_cp_wait();
    __syncthreads();
    if (act && more) {
      activate(ci + 1);
      __syncthreads();
    }
  }
  if (MODE != 2 && live) {
#pragma unroll
    for (int r = 0; r < R; r += 4)
      *reinterpret_cast<float4*>(S_g + (r >> 2) * gs) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
  }
}

// One thread per four neighbouring numbers of a request's memories: slice k's scratch memory becomes the memory at its
// start, and the slot's memory the one after the last slice. decay^len is a 64-bit power rounded once. Four slices' own
// memories are loaded ahead of the chain that needs them.
__global__ void __launch_bounds__(256) decay_pass_states_kernel(float* __restrict__ state, long long state_stride,
                                                                long long state_off, const int* __restrict__ cu_q,
                                                                const int* __restrict__ state_slots,
                                                                const float* __restrict__ decay, float* slice_S, int heads,
                                                                int dv, int d_pad, int slice_len, int max_slices) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int q_len = cu_q[s + 1] - cu_q[s];
  const long long per = (long long)heads * dv * d_pad;
  const long long e = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (e >= per || q_len <= 0) return;
  const double a = (double)decay[e / ((long long)dv * d_pad)];
  float4* slot = reinterpret_cast<float4*>(state + (size_t)state_slots[s] * state_stride + state_off + e);
  float4 S = *slot;
  const int slices = (q_len + slice_len - 1) / slice_len;
  const float a_full = (float)pow(a, (double)slice_len);
  const float a_last = (float)pow(a, (double)(q_len - (slices - 1) * slice_len));
  float4* mine = reinterpret_cast<float4*>(slice_S + (size_t)s * max_slices * per + e);
  const size_t step = (size_t)per / 4;
  for (int k0 = 0; k0 < slices; k0 += 4) {
    float4 own[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (k0 + j < slices) own[j] = mine[(size_t)(k0 + j) * step];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (k0 + j >= slices) break;
      const float f = k0 + j == slices - 1 ? a_last : a_full;
      mine[(size_t)(k0 + j) * step] = S;
      S.x = fmaf(f, S.x, own[j].x), S.y = fmaf(f, S.y, own[j].y), S.z = fmaf(f, S.z, own[j].z), S.w = fmaf(f, S.w, own[j].w);
    }
  }
  *slot = S;
}

// The activation on n ranges of columns of every row, in place.
__global__ void __launch_bounds__(256) decay_activate_kernel(float* __restrict__ proj, long long ld, int c0, int w0, int c1,
                                                             int w1, int c2, int w2, int act) {
  pdl_launch_dependents();
  pdl_wait();
  float* row = proj + (size_t)blockIdx.y * ld;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < w0 + w1 + w2; i += gridDim.x * blockDim.x) {
    const int c = i < w0 ? c0 + i : (i < w0 + w1 ? c1 + i - w0 : c2 + i - w0 - w1);
    row[c] = act_in(row[c], act);
  }
}

}  // namespace tmk

// proj: float, token t's row at proj + t * ld, q at q_col (heads x d), k at k_col, v at v_col (heads x dv); decay [heads]
// float; a request's memories ([heads][dv][d_pad] floats) start state_off floats into its slot of `state`
// (state_off and state_stride multiples of 4); y [T, heads * dv] float. mode 0: one walk per request. modes 1 and 2: the
// first and third pass over time slices of slice_len tokens, max_slices per request, through slice_S
// [n_seqs * max_slices] memories (float), with tm_decay_pass_states between.
extern "C" int tm_decay_memory(const float* proj, long long ld, int q_col, int k_col, int v_col, int act, const float* decay,
                               float* state, long long state_stride, long long state_off, const int* cu_q, const int* state_slots,
                               float* y, int n_seqs, int heads, int d, int dv, int mode, int slice_len, int max_slices,
                               float* slice_S, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || d < 1 || d > 512 || dv < 1 || (act != 0 && act != 1) || mode < 0 || mode > 2 || (state_stride & 3) ||
      (state_off & 3) || ((uintptr_t)state & 15))
    return TM_ERR_UNSUPPORTED_SHAPE;
  if (mode != 0 && (slice_len < 1 || max_slices < 1 || !slice_S || ((uintptr_t)slice_S & 15))) return TM_ERR_SCRATCH_TOO_SMALL;
  const tmk::DecayGeometry g = tmk::decay_geometry(heads, d, dv);
  const bool rows16 = !((uintptr_t)proj & 15) && !(ld & 3);
  const int vec = (rows16 && !(q_col & 3) && !(k_col & 3) && !(d & 3) ? 1 : 0) | (rows16 && !(v_col & 3) && !(dv & 3) ? 2 : 0);
  const size_t smem = sizeof(float) * 2 * tmk::kDecayChunk * (2 * (size_t)g.d_pad + g.cols);
  const dim3 grid(g.col_tiles, heads, n_seqs * (mode == 0 ? 1 : max_slices));
#define TM_DECAY_MODE(M_)                                                                                                  \
  {                                                                                                                        \
    auto kern = tmk::decay_memory_kernel<M_>;                                                                              \
    if (smem > 48 * 1024) {                                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
      if (e != cudaSuccess) return (int)e;                                                                                 \
    }                                                                                                                      \
    return tmk::launch_pdl(kern, grid, dim3(tmk::kDecayThreads), smem, stream, proj, ld, q_col, k_col, v_col, act, vec, decay, \
                           state, state_stride, state_off, cu_q, state_slots, y, heads, d, dv, g.parts, g.cols, slice_len, \
                           max_slices, slice_S);                                                                           \
  }
  if (mode == 0) TM_DECAY_MODE(0)
  if (mode == 1) TM_DECAY_MODE(1)
  TM_DECAY_MODE(2)
#undef TM_DECAY_MODE
}

// Between the two passes over time slices (see the top of the file).
extern "C" int tm_decay_pass_states(float* state, long long state_stride, long long state_off, const int* cu_q,
                                    const int* state_slots, const float* decay, float* slice_S, int n_seqs, int heads, int d,
                                    int dv, int slice_len, int max_slices, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || d < 1 || d > 512 || dv < 1 || slice_len < 1 || max_slices < 1 || !slice_S || (state_stride & 3) ||
      (state_off & 3))
    return TM_ERR_UNSUPPORTED_SHAPE;
  const tmk::DecayGeometry g = tmk::decay_geometry(heads, d, dv);
  const long long quads = g.floats / 4;
  return tmk::launch_pdl(tmk::decay_pass_states_kernel, dim3((unsigned)((quads + 255) / 256), n_seqs), dim3(256), 0, stream,
                         state, state_stride, state_off, cu_q, state_slots, decay, slice_S, heads, dv, g.d_pad, slice_len,
                         max_slices);
}

// act (1: silu) applied in place to the q, k (heads x d) and v (heads x dv) columns of all T rows of proj.
extern "C" int tm_decay_activate(float* proj, long long ld, int T, int q_col, int k_col, int v_col, int heads, int d, int dv,
                                 int act, cudaStream_t stream) {
  if (T <= 0 || act == 0) return 0;
  if (act != 1 || heads < 1 || d < 1 || dv < 1) return TM_ERR_UNSUPPORTED_SHAPE;
  const int total = 2 * heads * d + heads * dv;
  return tmk::launch_pdl(tmk::decay_activate_kernel, dim3((unsigned)std::min(64, (total + 255) / 256), T), dim3(256), 0, stream,
                         proj, ld, q_col, heads * d, k_col, heads * d, v_col, heads * dv, act);
}
