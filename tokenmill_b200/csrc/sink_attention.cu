// Grouped-query attention over a paged cache of [keys | values] rows, with the options a windowed design may combine:
// key and value heads of different sizes, a norm over the whole query / key projection, rotation of the first
// `rot_dims` dimensions of each head, a tanh cap on the scores, a sliding window that keeps the sequence's first
// tokens visible, a softmax with one more term of score 0 (a sink without a value), an output gate per head or per
// output number, and a query temperature that grows with the position. Each option is a parameter and may be switched off.
//
// tm_qk_norm_rope_write, one block per token, reads the token's row of a 32-bit projection
//   [q (H d) | k (G d) | v (G dv) | g (gate_cols)]        (g only with gate_out; k and v only with has_kv: a layer that
//                                                          reads another layer's keys and values has none)
// and writes: q, RMS-normed over all its H d numbers at once (weight wq; skipped when wq is null; with head_norm every
// head of q and k by its own root mean square instead, the weights then optional) and rotated, in the activation dtype; [k | v] to the token's cache row, k normed over its G d numbers (wk) and rotated; sigmoid(g) in
// 32-bit. With temp_every > 0 the query is multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) at position
// p (32-bit). The rotation pairs dimension i with i + rot_dims / 2 inside each head; angles come from 32-bit tables
// [positions, rot_dims / 2].
//
// tm_sink_attention: 32-bit arithmetic on CUDA cores for both dtypes. A tile is 32 consecutive (token, head in group)
// rows of one request and one key/value head; 8 warps x 4 rows. A query at position p sees key j <= p when
// p - j < window (window 0: every key) or j < keep_first. Keys are walked in tiles of 32 anchored at absolute positions
// 0, 32, 64, ...; tiles that no row of the block sees (between the kept first tokens and the window) are skipped. The
// order of every sum therefore depends only on the query's own position, never on how the request was cut into
// steps, on what else is in the batch, or on which pages hold the keys. The sink enters as the running maximum's and
// sum's starting values (score 0, weight 1, no value).
#include "common.cuh"

namespace tmk {

template <typename T>
__global__ void __launch_bounds__(256) qk_norm_rope_write_kernel(
    const float* __restrict__ proj, long long ld, int H, int G, int d, int dv, int rot_dims, const float* __restrict__ wq,
    const float* __restrict__ wk, float eps, const int* __restrict__ positions, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, int n_positions, const int* __restrict__ slot_map, T* __restrict__ q_out,
    T* __restrict__ cache, float* __restrict__ gate_out, int gate_cols, int has_kv, float temp_coef, int temp_every,
    int head_norm, int* __restrict__ error) {
  extern __shared__ __align__(16) float staged[];    // the token's q and k columns: read once, used three times; then,
                                                     // with a norm per head, one factor per head (H + G floats)
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * ld;
  const int nq = H * d, nk = has_kv ? G * d : 0, nv = has_kv ? G * dv : 0;
  const int pos = positions[t];
  const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
  const int half = rot_dims >> 1;
  if (rot_dims > 0 && (pos < 0 || pos >= n_positions)) {   // never read outside the tables: report instead
    if (threadIdx.x == 0) atomicExch(error, 31);
    return;
  }
  const float* ct = cos_t + (size_t)pos * half;
  const float* st = sin_t + (size_t)pos * half;

  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const float v = row[i];
    staged[i] = v;
    if (i < nq) sq += v * v;
    else sk += v * v;
  }
  float rq = 1.f, rk = 1.f;
  float* head_r = staged + nq + nk;
  if (head_norm) {          // every head of q and of k by its own root mean square (weights optional)
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int u = warp; u < H + (has_kv ? G : 0); u += n_warps) {
      const float* hp = staged + (size_t)u * d;
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) ss = fmaf(hp[i], hp[i], ss);
      ss = warp_sum(ss);
      if (lane == 0) head_r[u] = 1.0f / sqrtf(ss / (float)d + eps);
    }
    __syncthreads();
  } else {
    if (wq) rq = 1.0f / sqrtf(block_sum(sq, red) / (float)nq + eps);
    if (wk) rk = 1.0f / sqrtf(block_sum(sk, red) / (float)nk + eps);
    if (!wq && !wk) __syncthreads();
  }
  const int slot = slot_map ? slot_map[t] : -1;
  T* crow = slot >= 0 ? cache + (size_t)slot * (nk + nv) : nullptr;
  for (int idx = threadIdx.x; idx < nq + nk; idx += blockDim.x) {
    const bool is_q = idx < nq;
    if (!is_q && !crow) continue;
    const int i = is_q ? idx : idx - nq;
    const float* src = is_q ? staged : staged + nq;
    const float* w = is_q ? wq : wk;
    const float r = head_norm ? head_r[idx / d] : (is_q ? rq : rk);
    const int e = i % d;
    float v = src[i] * r * (w ? w[i] : 1.f);
    if (e < half) {
      const float o = src[i + half] * r * (w ? w[i + half] : 1.f);
      v = __fsub_rn(__fmul_rn(v, ct[e]), __fmul_rn(o, st[e]));
    } else if (e < rot_dims) {
      const float o = src[i - half] * r * (w ? w[i - half] : 1.f);
      v = __fadd_rn(__fmul_rn(v, ct[e - half]), __fmul_rn(o, st[e - half]));
    }
    if (is_q) q_out[(size_t)t * nq + i] = from_float<T>(v * temp);
    else crow[i] = from_float<T>(v);
  }
  if (crow)
    for (int i = threadIdx.x; i < nv; i += blockDim.x) crow[nk + i] = from_float<T>(row[nq + nk + i]);
  if (gate_out)
    for (int i = threadIdx.x; i < gate_cols; i += blockDim.x)
      gate_out[(size_t)t * gate_cols + i] = 1.0f / (1.0f + expf(-row[nq + nk + nv + i]));
}

constexpr int kSinkWarps = 8;
constexpr int kSinkRowsPerWarp = 4;
constexpr int kSinkTileRows = kSinkWarps * kSinkRowsPerWarp;   // 32
constexpr int kSinkKeyTile = 32;

template <typename T, int NDV>
__global__ void __launch_bounds__(kSinkWarps * 32) sink_attention_kernel(
    const T* __restrict__ q, const T* __restrict__ cache, int row_width, int v_off, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_before, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_row0, const float* __restrict__ gate, T* __restrict__ out, int H, int G, int d, int dv,
    int page_size, float scale, float softcap, int window, int keep_first, int sink, int gate_wide,
    float* __restrict__ cross_out) {
  extern __shared__ __align__(16) float smem[];
  const int KS = d + 1;                           // padded key row: lanes read different rows, same column
  float* qs = smem;                               // [32][d]
  float* ks = qs + kSinkTileRows * d;             // [32][d + 1]
  float* vs = ks + kSinkKeyTile * KS;             // [32][dv]

  pdl_launch_dependents();
  pdl_wait();
  const int s = tile_seq[blockIdx.x];
  const int row0 = tile_row0[blockIdx.x];
  // cross_out: blockIdx.y = key head * G + value head, and the head's weights meet the values of that value head
  const int kvh = cross_out ? blockIdx.y / G : blockIdx.y;
  const int vh = cross_out ? blockIdx.y - kvh * G : kvh;
  const int Gq = H / G;
  const int q_start = cu_q[s];
  const int q_len = cu_q[s + 1] - q_start;
  const int before = kv_before[s];
  const int n_rows = q_len * Gq;
  if (row0 >= n_rows) return;
  const int row_end = min(row0 + kSinkTileRows, n_rows);
  const int p_min = before + row0 / Gq;
  const int p_max = before + (row_end - 1) / Gq;
  const int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;     // the earliest key inside any row's window
  const int j_hi = p_max;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = block_table + (size_t)s * bt_stride;

  for (int idx = tid; idx < kSinkTileRows * d; idx += blockDim.x) {
    const int r = idx / d, e = idx - r * d;
    const int row = row0 + r;
    float v = 0.f;
    if (row < n_rows) v = to_float(q[((size_t)(q_start + row / Gq) * H + kvh * Gq + row % Gq) * d + e]);
    qs[idx] = v;
  }

  // a warp's rows are warp, warp + 8, ...: a step of few rows (decoding) spreads them over the warps
  float m[kSinkRowsPerWarp], l[kSinkRowsPerWarp], acc[kSinkRowsPerWarp][NDV];
  int p_row[kSinkRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kSinkRowsPerWarp; ++i) {
    m[i] = sink ? 0.f : -INFINITY;
    l[i] = sink ? 1.f : 0.f;
#pragma unroll
    for (int dd = 0; dd < NDV; ++dd) acc[i][dd] = 0.f;
    const int row = row0 + i * kSinkWarps + warp;
    p_row[i] = row < n_rows ? before + row / Gq : -1;
  }
  const bool warp_idle = p_row[0] < 0;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;

  for (int kt = 0; kt <= j_hi; kt += kSinkKeyTile) {
    if (kt >= keep_first && kt + kSinkKeyTile <= j_lo) {       // nobody sees this tile: jump to the window's first
      kt = (j_lo / kSinkKeyTile) * kSinkKeyTile - kSinkKeyTile;
      continue;
    }
    __syncthreads();
    {   // eight threads a key row: one page lookup each, then loads that do not wait on one another
      const int jj = tid >> 3, part = tid & 7;
      const int j = kt + jj;
      const bool seen = j <= j_hi && (j >= j_lo || j < keep_first);
      const T* src = cache;
      if (seen) src += ((size_t)table[j / page_size] * page_size + (j % page_size)) * row_width;
      const T* kp = src + kvh * d;
      const T* vp = src + v_off + vh * dv;
      for (int e = part; e < d; e += 8) ks[jj * KS + e] = seen ? to_float(kp[e]) : 0.f;
      for (int e = part; e < dv; e += 8) vs[jj * dv + e] = seen ? to_float(vp[e]) : 0.f;
    }
    __syncthreads();
    if (warp_idle) continue;

    float sc[kSinkRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kSinkRowsPerWarp; ++i) sc[i] = 0.f;
    const float* krow = ks + lane * KS;
    for (int e = 0; e < d; ++e) {
      const float kk = krow[e];
#pragma unroll
      for (int i = 0; i < kSinkRowsPerWarp; ++i) sc[i] = fmaf(qs[(i * kSinkWarps + warp) * d + e], kk, sc[i]);
    }
    const int j = kt + lane;
    float p[kSinkRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kSinkRowsPerWarp; ++i) {
      const int pr = p_row[i];
      const bool ok = j <= pr && (window <= 0 || pr - j < window || j < keep_first);
      float sv = sc[i] * scale;
      if (softcap > 0.f) sv = softcap * tanhf(sv * inv_cap);
      sv = ok ? sv : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(sv));
      float corr = 1.f, pv = 0.f;
      if (m_new != -INFINITY) {
        corr = expf(m[i] - m_new);
        pv = ok ? expf(sv - m_new) : 0.f;
      }
      l[i] = l[i] * corr + warp_sum(pv);
      m[i] = m_new;
      p[i] = pv;
#pragma unroll
      for (int dd = 0; dd < NDV; ++dd) acc[i][dd] *= corr;
    }
    for (int jj = 0; jj < kSinkKeyTile; ++jj) {
      float vv[NDV];
#pragma unroll
      for (int dd = 0; dd < NDV; ++dd) {
        const int e = lane + 32 * dd;
        vv[dd] = e < dv ? vs[jj * dv + e] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < kSinkRowsPerWarp; ++i) {
        const float pj = __shfl_sync(0xffffffffu, p[i], jj);
#pragma unroll
        for (int dd = 0; dd < NDV; ++dd) acc[i][dd] = fmaf(pj, vv[dd], acc[i][dd]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < kSinkRowsPerWarp; ++i) {
    const int row = row0 + i * kSinkWarps + warp;
    if (row >= n_rows) continue;
    const int tok = q_start + row / Gq, head = kvh * Gq + row % Gq;
    float f = l[i] > 0.f ? 1.0f / l[i] : 0.f;
    if (cross_out) {
      float* o32 = cross_out + (((size_t)tok * H + head) * G + vh) * dv;
#pragma unroll
      for (int dd = 0; dd < NDV; ++dd) {
        const int e = lane + 32 * dd;
        if (e < dv) o32[e] = acc[i][dd] * f;
      }
      continue;
    }
    if (gate && !gate_wide) f *= gate[(size_t)tok * H + head];
    T* o = out + ((size_t)tok * H + head) * dv;
    const float* gw = (gate && gate_wide) ? gate + ((size_t)tok * H + head) * dv : nullptr;
#pragma unroll
    for (int dd = 0; dd < NDV; ++dd) {
      const int e = lane + 32 * dd;
      if (e < dv) o[e] = from_float<T>(acc[i][dd] * f * (gw ? gw[e] : 1.0f));
    }
  }
}

template <typename T>
int launch_sink_attention(const void* q, const void* cache, int row_width, int v_off, const int* block_table, int bt_stride,
                          const int* cu_q, const int* kv_before, const int* tile_seq, const int* tile_row0, int n_tiles,
                          const float* gate, void* out, int H, int G, int d, int dv, int page_size, float scale,
                          float softcap, int window, int keep_first, int sink, int gate_wide, float* cross_out,
                          cudaStream_t stream) {
  const size_t smem = ((size_t)kSinkTileRows * d + (size_t)kSinkKeyTile * (d + 1) + (size_t)kSinkKeyTile * dv) * sizeof(float);
  if (smem > 220 * 1024 || dv > 256 || H % G) return TM_ERR_UNSUPPORTED_SHAPE;
  const int nd = (dv + 31) / 32;
#define TM_SINK_CASE(NDV)                                                                                         \
  case NDV: {                                                                                                     \
    auto kern = sink_attention_kernel<T, NDV>;                                                                    \
    if (smem > 48 * 1024) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      if (e != cudaSuccess) return (int)e;                                                                        \
    }                                                                                                             \
    return launch_pdl(kern, dim3(n_tiles, cross_out ? G * G : G), dim3(kSinkWarps * 32), smem, stream, (const T*)q, \
                      (const T*)cache, row_width, v_off, block_table, bt_stride, cu_q, kv_before, tile_seq, tile_row0, gate, \
                      (T*)out, H, G, d, dv, page_size, scale, softcap, window, keep_first, sink, gate_wide, cross_out); \
  }
  switch (nd) {
    TM_SINK_CASE(1) TM_SINK_CASE(2) TM_SINK_CASE(3) TM_SINK_CASE(4) TM_SINK_CASE(5) TM_SINK_CASE(6) TM_SINK_CASE(7)
    TM_SINK_CASE(8)
    default: return TM_ERR_UNSUPPORTED_SHAPE;
  }
#undef TM_SINK_CASE
}

}  // namespace tmk

// proj: float, token t's row at proj + t * ld; wq [H d], wk [G d] float or null; cos/sin [n_positions, rot_dims / 2] float;
// slot_map [T] or null (negative: not cached); q_out [T, H d]; cache [slots, G d + G dv]; gate_out [T, gate_cols] float or
// null; has_kv 0: the row is [q | g] only; temp_every > 0: the query temperature.
extern "C" int tm_qk_norm_rope_write(int dtype, const float* proj, long long ld, int H, int G, int d, int dv, int rot_dims,
                                     const float* wq, const float* wk, float eps, const int* positions, const float* cos_t,
                                     const float* sin_t, int n_positions, const int* slot_map, void* q_out, void* cache,
                                     float* gate_out, int gate_cols, int has_kv, float temp_coef, int temp_every, int head_norm,
                                     int T_rows, int* error, cudaStream_t stream) {
  if (T_rows <= 0) return 0;
  if (rot_dims % 2 || rot_dims > d || rot_dims < 0 || H <= 0 || G <= 0 || temp_every < 0) return TM_ERR_UNSUPPORTED_SHAPE;
  if (!has_kv && (cache || wk)) return TM_ERR_UNSUPPORTED_SHAPE;
  const size_t smem = ((size_t)(H + G) * d + (head_norm ? H + G : 0)) * sizeof(float);
  if (smem > 200 * 1024) return TM_ERR_UNSUPPORTED_SHAPE;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(tmk::qk_norm_rope_write_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tmk::qk_norm_rope_write_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_pdl(tmk::qk_norm_rope_write_kernel<float>, dim3(T_rows), dim3(256), smem, stream, proj, ld, H, G, d, dv,
                           rot_dims, wq, wk, eps, positions, cos_t, sin_t, n_positions, slot_map, (float*)q_out,
                           (float*)cache, gate_out, gate_cols, has_kv, temp_coef, temp_every, head_norm, error);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_pdl(tmk::qk_norm_rope_write_kernel<__nv_bfloat16>, dim3(T_rows), dim3(256), smem, stream, proj, ld, H, G,
                           d, dv, rot_dims, wq, wk, eps, positions, cos_t, sin_t, n_positions, slot_map,
                           (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, gate_out, gate_cols, has_kv, temp_coef, temp_every,
                           head_norm, error);
  return TM_ERR_BAD_DTYPE;
}

// q [T, H, d]; cache [pages, page_size, row_width] with head g's key at g * d and its value at v_off + g * dv; tiles of 32
// (token, head in group) rows; gate [T, H] float (gate_wide: [T, H, dv]) or null; out [T, H, dv]. cross_out [T, H, G, dv]
// float (then out and gate are not used): every head's softmax weights applied to the values of each of the G value heads.
extern "C" int tm_sink_attention(int dtype, const void* q, const void* cache, int row_width, int v_off,
                                 const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                                 const int* tile_seq, const int* tile_row0, int n_tiles, const float* gate, void* out, int H,
                                 int G, int d, int dv, int page_size, float scale, float softcap, int window, int keep_first,
                                 int sink, int gate_wide, float* cross_out, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (cross_out && gate) return TM_ERR_UNSUPPORTED_SHAPE;
  if (dtype == TM_DTYPE_F32)
    return tmk::launch_sink_attention<float>(q, cache, row_width, v_off, block_table, bt_stride, cu_q, kv_before, tile_seq,
                                             tile_row0, n_tiles, gate, out, H, G, d, dv, page_size, scale, softcap, window,
                                             keep_first, sink, gate_wide, cross_out, stream);
  if (dtype == TM_DTYPE_BF16)
    return tmk::launch_sink_attention<__nv_bfloat16>(q, cache, row_width, v_off, block_table, bt_stride, cu_q, kv_before,
                                                     tile_seq, tile_row0, n_tiles, gate, out, H, G, d, dv, page_size, scale,
                                                     softcap, window, keep_first, sink, gate_wide, cross_out, stream);
  return TM_ERR_BAD_DTYPE;
}
