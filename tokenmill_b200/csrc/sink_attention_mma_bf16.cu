// The attention of sink_attention.cu on tensor cores (bfloat16 in, float32 scores, softmax and sums), for key heads and
// value heads of 32, 64 or 128 (each its own size). Same semantics: a cache row per token holding all key heads and then
// all value heads; query head h reads key/value head h / (H / G); a query at position p sees key j <= p when
// p - j < window (window 0: every key) or j < keep_first; scores are scaled, then capped (cap tanh(s / cap)); the
// softmax may carry a sink of score 0 without a value; each head's output may be multiplied by a gate.
//
// A block takes 64 consecutive (token, head in group) rows of one request and one key/value head: four warps of 16 rows.
// Keys stream through shared memory in blocks of 64 anchored at absolute positions 0, 64, 128, ... (a cp.async ring; one
// page lookup per key row): first the blocks that hold kept first tokens below the window, then the blocks from the
// window's first key on; what lies between is never read. Because the blocks are anchored, a row's sums run in the same
// order however the request was cut into steps. A warp multiplies its rows with the whole block (ldmatrix +
// mma.sync m16n8k16), keeps maximum, sum and output in registers, and adds P V with V read through ldmatrix.trans. The
// window bounds a row's keys, so a prompt's tile is never cut into key chunks. A step of few rows (decoding) deals a
// tile's key blocks out over `n_splits` blocks of the grid (block z takes key blocks z, z + n_splits, ...; the sink
// belongs to z = 0); each leaves unnormalised sums with its maximum and denominator, and tm_sink_attention_combine
// merges them in the order of z. tanh is taken as 1 - 2 / (exp(2x) + 1) in 32-bit (absolute error of the order of
// 1e-7); P is rounded to bfloat16 for the second product.
#include "mma_util.cuh"

namespace tmk {

constexpr int kSmBM = 64;        // rows per block
constexpr int kSmBN = 64;        // keys per stage
constexpr int kSmWarps = 4;

template <int CH> __device__ __forceinline__ int sm_swz(int row, int c) {
  if constexpr (CH >= 8) return c ^ (row & 7);
  else return c ^ ((row >> 1) & 3);
}

template <int DK, int DV, int STAGES>
__global__ void __launch_bounds__(kSmWarps * 32) sink_attention_mma_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, int row_width, int v_off,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_before,
    const int* __restrict__ tile_seq, const int* __restrict__ tile_row0, const float* __restrict__ gate,
    __nv_bfloat16* __restrict__ out, int H, int G, int page_size, float scale, float softcap, int window, int keep_first,
    int sink, int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml, int gate_wide,
    float* __restrict__ cross_out) {
  constexpr int THREADS = kSmWarps * 32;
  constexpr int CHK = DK / 8, CHV = DV / 8;     // 16-byte chunks per key / value row
  constexpr int TPR = THREADS / kSmBN;          // threads that share one key row when loading (2)
  constexpr int KS = DK / 16;
  constexpr int NT = DV / 8;
  constexpr int K_BYTES = kSmBN * DK * 2, V_BYTES = kSmBN * DV * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cpair = (lane & 3) * 2;

  pdl_launch_dependents();
  pdl_wait();
  // cross_out: blockIdx.y = key head * G + value head, and the head's weights meet the values of that value head
  const int s = tile_seq[blockIdx.x], row0 = tile_row0[blockIdx.x];
  const int kvh = cross_out ? blockIdx.y / G : blockIdx.y;
  const int vh = cross_out ? blockIdx.y - kvh * G : kvh;
  const int Gq = H / G;
  const int q_start = cu_q[s], q_len = cu_q[s + 1] - q_start, before = kv_before[s];
  const int n_rows = min(kSmBM, q_len * Gq - row0);
  if (n_rows <= 0) return;
  const int p_min = before + row0 / Gq, p_max = before + (row0 + n_rows - 1) / Gq;
  const int j_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  const int j_hi = p_max;
  const int keep = window > 0 ? keep_first : 0;
  const int keep_end = min(keep, j_lo);                           // kept keys that lie below the window's first key
  const int n_keep = (keep_end + kSmBN - 1) / kSmBN;              // blocks 0 .. n_keep - 1 hold them
  const int kb_first = max(n_keep * kSmBN, (j_lo / kSmBN) * kSmBN);
  const int all_blocks = n_keep + (j_hi >= kb_first ? (j_hi - kb_first) / kSmBN + 1 : 0);
  const int split = blockIdx.z;
  const int n_blocks = all_blocks > split ? (all_blocks - split + n_splits - 1) / n_splits : 0;   // this block's share
  const int* table = block_table + (size_t)s * bt_stride;

  uint32_t qa[KS][4];
  int p_row[2];
  size_t o_row[2];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = warp * 16 + (lane >> 2) + hh * 8;
    const bool ok = r < n_rows;
    const int row = row0 + (ok ? r : 0);
    const int tok = row / Gq, g = row - tok * Gq;
    o_row[hh] = (size_t)(q_start + tok) * H + kvh * Gq + g;
    p_row[hh] = ok ? before + tok : -1;
    const __nv_bfloat16* qr = q + o_row[hh] * DK;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c = ks * 16 + cpair;
      qa[ks][hh] = ok ? *reinterpret_cast<const uint32_t*>(qr + c) : 0u;
      qa[ks][2 + hh] = ok ? *reinterpret_cast<const uint32_t*>(qr + c + 8) : 0u;
    }
  }
  const int w_first = min(warp * 16, n_rows - 1), w_last = min(warp * 16 + 15, n_rows - 1);
  const bool warp_has_rows = warp * 16 < n_rows;
  const int wp_lo = before + (row0 + w_first) / Gq, wp_hi = before + (row0 + w_last) / Gq;
  const int w_key_lo = window > 0 ? max(0, wp_lo - window + 1) : 0;        // first window key any row of the warp sees
  const int w_full_lo = window > 0 ? max(0, wp_hi - window + 1) : 0;       // first window key every row sees

  // log2 units throughout: y = score * scale * log2(e), capped if asked
  constexpr float kLog2e = 1.4426950408889634f;
  const float plain_mul = scale * kLog2e;
  const float cap_in = softcap > 0.f ? scale / softcap * 2.0f * kLog2e : 0.f;   // exp2 argument of exp(2 s / cap)
  const float cap_out = softcap * kLog2e;

  float m_run[2], l_run[2];
  float o[NT][4];
  m_run[0] = m_run[1] = (sink && split == 0) ? 0.f : -INFINITY;
  l_run[0] = l_run[1] = (sink && split == 0) ? 1.f : 0.f;
#pragma unroll
  for (int t = 0; t < NT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

  auto block_start = [&](int i) {               // the i-th key block of this block's share
    const int b = split + i * n_splits;
    return b < n_keep ? b * kSmBN : kb_first + (b - n_keep) * kSmBN;
  };
  auto load_block = [&](int stage, int kb) {
    const uint32_t k_dst = smem_base + stage * (K_BYTES + V_BYTES), v_dst = k_dst + K_BYTES;
    const int row = tid / TPR, part = tid - row * TPR;
    const int j = kb + row;
    const bool ok = j <= j_hi && (j >= j_lo || j < keep);
    size_t src = 0;
    if (ok) {
      const int page = table[j / page_size];
      src = ((size_t)page * page_size + (j % page_size)) * row_width;
    }
    const __nv_bfloat16* kp = cache + src + kvh * DK;
    const __nv_bfloat16* vp = cache + src + v_off + vh * DV;
#pragma unroll
    for (int i = 0; i < CHK / TPR; ++i) {
      const int c = part * (CHK / TPR) + i;
      cp_async16(k_dst + row * (DK * 2) + (sm_swz<CHK>(row, c) << 4), kp + c * 8, ok);
    }
#pragma unroll
    for (int i = 0; i < CHV / TPR; ++i) {
      const int c = part * (CHV / TPR) + i;
      cp_async16(v_dst + row * (DV * 2) + (sm_swz<CHV>(row, c) << 4), vp + c * 8, ok);
    }
  };

#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (i < n_blocks) load_block(i, block_start(i));
    cp_async_commit();
  }
  for (int b = 0; b < n_blocks; ++b) {
    cp_async_wait<STAGES - 2>();             // block b has landed (this thread's copies)
    __syncthreads();                         // ... everyone's; and block b - 1 is fully consumed
    {
      const int nb = b + STAGES - 1;
      if (nb < n_blocks) load_block(nb % STAGES, block_start(nb));
      cp_async_commit();
    }
    const int kb = block_start(b);
    const int stage = b % STAGES;
    // nothing of this block visible to this warp: behind its rows, or between its kept tokens and its windows
    if (!warp_has_rows || kb > wp_hi || (kb + kSmBN - 1 < w_key_lo && kb >= keep)) continue;

    const uint32_t k_base = smem_base + stage * (K_BYTES + V_BYTES), v_base = k_base + K_BYTES;
    float sc[8][4];
#pragma unroll
    for (int t = 0; t < 8; ++t) sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
    {
      const int krow = (lane & 7) + ((lane >> 4) << 3);
      const int csel = (lane >> 3) & 1;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const int key = kk * 16 + krow;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(k_base + key * (DK * 2) + (sm_swz<CHK>(key, 2 * ks + csel) << 4), b0, b1, b2, b3);
          mma_bf16_16816(sc[2 * kk], qa[ks], b0, b1);
          mma_bf16_16816(sc[2 * kk + 1], qa[ks], b2, b3);
        }
      }
    }
    // every key of the block visible to every row of the warp: no mask needed
    const bool all_seen = kb + kSmBN - 1 <= wp_lo && (kb >= w_full_lo || kb + kSmBN - 1 < keep);
    float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float y;
        if (softcap > 0.f) {
          const float ex = exp2f(sc[t][e] * cap_in);
          y = cap_out * (1.0f - __fdividef(2.0f, ex + 1.0f));
        } else {
          y = sc[t][e] * plain_mul;
        }
        if (!all_seen) {
          const int j = kb + t * 8 + cpair + (e & 1);
          const int p = p_row[e >> 1];
          if (!(j <= p && (window <= 0 || j > p - window || j < keep))) y = -INFINITY;
        }
        sc[t][e] = y;
        if (e < 2) tmax0 = fmaxf(tmax0, y);
        else tmax1 = fmaxf(tmax1, y);
      }
    tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
    tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
    const float mn0 = fmaxf(m_run[0], tmax0), mn1 = fmaxf(m_run[1], tmax1);
    const float corr0 = mn0 == -INFINITY ? 1.f : exp2f(m_run[0] - mn0);
    const float corr1 = mn1 == -INFINITY ? 1.f : exp2f(m_run[1] - mn1);
    const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
    float ps0 = 0.f, ps1 = 0.f;
    uint32_t pa[4][4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      float p[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[h][e] = exp2f(sc[2 * kk + h][e] - base0);              // masked entries are -inf: 0
          p[h][2 + e] = exp2f(sc[2 * kk + h][2 + e] - base1);
          ps0 += p[h][e];
          ps1 += p[h][2 + e];
        }
      pa[kk][0] = pack_bf16(p[0][0], p[0][1]);
      pa[kk][1] = pack_bf16(p[0][2], p[0][3]);
      pa[kk][2] = pack_bf16(p[1][0], p[1][1]);
      pa[kk][3] = pack_bf16(p[1][2], p[1][3]);
    }
    ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1);
    ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
    ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1);
    ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
    l_run[0] = l_run[0] * corr0 + ps0;
    l_run[1] = l_run[1] * corr1 + ps1;
    m_run[0] = mn0;
    m_run[1] = mn1;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      o[t][0] *= corr0;
      o[t][1] *= corr0;
      o[t][2] *= corr1;
      o[t][3] *= corr1;
    }
    {
      const int krow = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int csel = lane >> 4;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int key = kk * 16 + krow;
#pragma unroll
        for (int dt = 0; dt < NT / 2; ++dt) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(v_base + key * (DV * 2) + (sm_swz<CHV>(key, 2 * dt + csel) << 4), b0, b1, b2, b3);
          mma_bf16_16816(o[2 * dt], pa[kk], b0, b1);
          mma_bf16_16816(o[2 * dt + 1], pa[kk], b2, b3);
        }
      }
    }
  }
  cp_async_wait<0>();

  if (n_splits > 1) {                           // one of several: sums, maximum (log2 units) and denominator
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      if (p_row[hh] < 0) continue;
      const int r = warp * 16 + (lane >> 2) + hh * 8;
      const size_t prow = (((size_t)blockIdx.x * gridDim.y + blockIdx.y) * n_splits + split) * kSmBM + r;
      float* dst = part_o + prow * DV;
#pragma unroll
      for (int t = 0; t < NT; ++t)
        *reinterpret_cast<float2*>(dst + t * 8 + cpair) = make_float2(o[t][2 * hh], o[t][2 * hh + 1]);
      if ((lane & 3) == 0) *reinterpret_cast<float2*>(part_ml + prow * 2) = make_float2(m_run[hh], l_run[hh]);
    }
    return;
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    if (p_row[hh] < 0) continue;
    float f = l_run[hh] > 0.f ? 1.0f / l_run[hh] : 0.f;
    if (cross_out) {
      float* dst32 = cross_out + (o_row[hh] * G + vh) * DV;
#pragma unroll
      for (int t = 0; t < NT; ++t)
        *reinterpret_cast<float2*>(dst32 + t * 8 + cpair) = make_float2(o[t][2 * hh] * f, o[t][2 * hh + 1] * f);
      continue;
    }
    if (gate && !gate_wide) f *= gate[o_row[hh]];
    __nv_bfloat16* dst = out + o_row[hh] * DV;
    const float* gw = (gate && gate_wide) ? gate + o_row[hh] * DV : nullptr;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      float g0 = 1.f, g1 = 1.f;
      if (gw) { g0 = gw[t * 8 + cpair]; g1 = gw[t * 8 + cpair + 1]; }
      *reinterpret_cast<uint32_t*>(dst + t * 8 + cpair) = pack_bf16(o[t][2 * hh] * f * g0, o[t][2 * hh + 1] * f * g1);
    }
  }
}

// Merges the partial results of a tile's key splits in the order of the splits; one block per (tile, key/value head),
// a warp per row in turn.
__global__ void __launch_bounds__(256) sink_attention_combine_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ cu_q,
    const int* __restrict__ tile_seq, const int* __restrict__ tile_row0, const float* __restrict__ gate,
    __nv_bfloat16* __restrict__ out, int H, int G, int dv, int n_splits, int gate_wide, float* __restrict__ cross_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = tile_seq[blockIdx.x], row0 = tile_row0[blockIdx.x];
  const int kvh = cross_out ? blockIdx.y / G : blockIdx.y;
  const int vh = cross_out ? blockIdx.y - kvh * G : kvh;
  const int Gq = H / G;
  const int q_start = cu_q[s], q_len = cu_q[s + 1] - q_start;
  const int n_rows = min(kSmBM, q_len * Gq - row0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t base = ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * n_splits;
  for (int r = warp; r < n_rows; r += 8) {
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, part_ml[((base + z) * kSmBM + r) * 2]);
    float L = 0.f;
    for (int z = 0; z < n_splits; ++z) {
      const float* ml = part_ml + ((base + z) * kSmBM + r) * 2;
      if (ml[0] != -INFINITY) L += ml[1] * exp2f(ml[0] - M);
    }
    const int row = row0 + r;
    const size_t o_row = (size_t)(q_start + row / Gq) * H + kvh * Gq + row % Gq;
    float f = L > 0.f ? 1.0f / L : 0.f;
    if (gate && !gate_wide) f *= gate[o_row];
    const float* gw = (gate && gate_wide) ? gate + o_row * dv : nullptr;
    for (int e = lane; e < dv; e += 32) {
      float acc = 0.f;
      for (int z = 0; z < n_splits; ++z) {
        const float mz = part_ml[((base + z) * kSmBM + r) * 2];
        if (mz != -INFINITY) acc += part_o[((base + z) * kSmBM + r) * dv + e] * exp2f(mz - M);
      }
      if (cross_out) cross_out[(o_row * G + vh) * dv + e] = acc * f;
      else out[o_row * dv + e] = __float2bfloat16_rn(acc * f * (gw ? gw[e] : 1.0f));
    }
  }
}

template <int DK, int DV>
int launch_sink_attention_mma(const void* q, const void* cache, int row_width, int v_off, const int* block_table,
                              int bt_stride, const int* cu_q, const int* kv_before, const int* tile_seq,
                              const int* tile_row0, int n_tiles, const float* gate, void* out, int H, int G, int page_size,
                              float scale, float softcap, int window, int keep_first, int sink, int n_splits, float* part_o,
                              float* part_ml, int gate_wide, float* cross_out, cudaStream_t stream) {
  constexpr int STAGES = (DK + DV) >= 256 ? 2 : 3;
  const int smem = STAGES * kSmBN * (DK + DV) * 2;
  auto kern = sink_attention_mma_kernel<DK, DV, STAGES>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int gy = cross_out ? G * G : G;
  const int st = launch_pdl(kern, dim3(n_tiles, gy, n_splits), dim3(kSmWarps * 32), (size_t)smem, stream,
                            (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, row_width, v_off, block_table, bt_stride, cu_q,
                            kv_before, tile_seq, tile_row0, gate, (__nv_bfloat16*)out, H, G, page_size, scale, softcap, window,
                            keep_first, sink, n_splits, part_o, part_ml, gate_wide, cross_out);
  if (st != 0 || n_splits == 1) return st;
  return launch_pdl(sink_attention_combine_kernel, dim3(n_tiles, gy), dim3(256), 0, stream, (const float*)part_o,
                    (const float*)part_ml, cu_q, tile_seq, tile_row0, gate, (__nv_bfloat16*)out, H, G, DV, n_splits, gate_wide,
                    cross_out);
}

}  // namespace tmk

// q [T, H, d] bfloat16; cache [pages, page_size, row_width] bfloat16 with head g's key at g * d and its value at
// v_off + g * dv (row_width and v_off multiples of 8); tiles of 64 (token, head in group) rows of one request; gate
// [T, H] float (gate_wide: [T, H, dv]) or null; out [T, H, dv] bfloat16. d and dv each 32, 64 or 128; the scale positive. n_splits > 1: a
// tile's key blocks are dealt out over that many blocks, through part_o [n_tiles * G * n_splits, 64, dv] and part_ml
// [n_tiles * G * n_splits, 64, 2] float, and merged by a second launch. cross_out [T, H, G, dv] float (then out and gate
// are not used, and the partial results have G times the rows): every head's softmax weights applied to the values of
// each of the G value heads.
extern "C" int tm_sink_attention_mma_bf16(const void* q, const void* cache, int row_width, int v_off,
                                          const int* block_table, int bt_stride, const int* cu_q, const int* kv_before,
                                          const int* tile_seq, const int* tile_row0, int n_tiles, const float* gate,
                                          void* out, int H, int G, int d, int dv, int page_size, float scale, float softcap,
                                          int window, int keep_first, int sink, int n_splits, float* part_o, float* part_ml,
                                          int gate_wide, float* cross_out, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (cross_out && gate) return TM_ERR_UNSUPPORTED_SHAPE;
  if (n_splits < 1 || (n_splits > 1 && (!part_o || !part_ml))) return TM_ERR_SCRATCH_TOO_SMALL;
  if (G <= 0 || H % G || page_size <= 0 || (row_width & 7) || (v_off & 7) || !(scale > 0.f)) return TM_ERR_UNSUPPORTED_SHAPE;
#define TM_SM_CASE(DKK, DVV)                                                                                          \
  if (d == DKK && dv == DVV)                                                                                          \
    return tmk::launch_sink_attention_mma<DKK, DVV>(q, cache, row_width, v_off, block_table, bt_stride, cu_q, kv_before, \
                                                    tile_seq, tile_row0, n_tiles, gate, out, H, G, page_size, scale, softcap, \
                                                    window, keep_first, sink, n_splits, part_o, part_ml, gate_wide, cross_out, stream);
  TM_SM_CASE(32, 32) TM_SM_CASE(32, 64) TM_SM_CASE(32, 128) TM_SM_CASE(64, 32) TM_SM_CASE(64, 64) TM_SM_CASE(64, 128)
  TM_SM_CASE(128, 32) TM_SM_CASE(128, 64) TM_SM_CASE(128, 128)
#undef TM_SM_CASE
  return TM_ERR_UNSUPPORTED_SHAPE;
}
