// Device body of the tensor-core split pass over un-quantized 16-bit K/V (see paged_decode_mma.cu for the data flow).
#pragma once

#include "decode_core.cuh"
#include "decode_params.cuh"
#include "mma_utils.cuh"

namespace anna {

constexpr int kMmaWarps = 4;
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kTileTokens = 16;

template <int D>
struct MmaCfg {
  static constexpr int kSteps = D / 16;                 // k-steps of Q.K and m-tiles of P.V
  static constexpr int kChunksPerRow = D / 8;           // 16-byte chunks per token row
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = kTileTokens * kRowBytes;
  static constexpr int kStages = 2;
  static constexpr int kCopiesPerLane = kTileTokens * kChunksPerRow / 32;
  static constexpr int kRowsPerCopy = 32 / kChunksPerRow > 0 ? 32 / kChunksPerRow : 1;
  static constexpr int kWarpSmem = kStages * 2 * kTileBytes;
  static constexpr int kFlagBytes = kMmaWarps * 16;
  static constexpr int kSmemBytes = kMmaWarps * kWarpSmem + kFlagBytes;
  static constexpr int kMinBlocks = D >= 256 ? 1 : (D == 128 ? 3 : 4);
};

// Split pass over tokens [t0, t1) of (row b, kv head kvh, query heads g0 .. g0 + g_count) for one CTA of kMmaThreads
// threads; the partial goes to split-K slot `slot`, and with a fused merge it counts as one of the `active_chunks`
// arrivals on counters[counter_index].
// Token t lives at element offset: paged -> page_table / block_size; ring_len > 0 -> (t % ring_len) * D; else
// t * kv_stride_t, all relative to the (row, kv head) base the caller put into p.key / p.value.
template <typename T, int D>
__device__ __forceinline__ void dense_split_mma_body(const DenseDecodeParams& p, uint8_t* smem_raw, int b, int kvh,
                                                     int g0, int g_count, int t0, int t1, int slot,
                                                     int active_chunks, int64_t counter_index) {
  using Cfg = MmaCfg<D>;
  const int num_tiles = (t1 - t0 + kTileTokens - 1) / kTileTokens;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2;
  const int tig = lane & 3;
  const int hq0 = kvh * p.groups + g0;

  // ---- Q^T fragments: b0 = Q[head gid][16s + 2tig .. +1], b1 = Q[head gid][16s + 8 + 2tig .. +1] ---------------------
  uint32_t qf[Cfg::kSteps][2];
  {
    const T* q_row = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b + (int64_t)(hq0 + gid) * p.q_stride_h;
#pragma unroll
    for (int s = 0; s < Cfg::kSteps; ++s) {
      if (gid < g_count) {
        qf[s][0] = *reinterpret_cast<const uint32_t*>(q_row + 16 * s + 2 * tig);
        qf[s][1] = *reinterpret_cast<const uint32_t*>(q_row + 16 * s + 8 + 2 * tig);
      } else {
        qf[s][0] = 0u;
        qf[s][1] = 0u;
      }
    }
  }

  const bool paged = p.page_table != nullptr;
  const int ring_len = p.ring_len;
  // "contiguous tile": the 16 token rows of a tile sit back to back in memory (page size a multiple of 16, or a dense
  // tensor with token stride D); otherwise every row is located on its own.
  const bool tile_contiguous =
      paged ? (p.block_size % kTileTokens == 0) : (ring_len > 0 ? false : p.kv_stride_t == D);
  const uint32_t block_size = (uint32_t)p.block_size;
  const int block_shift = p.block_shift;
  const T* k_base;
  const T* v_base;
  if (paged) {
    const int64_t head_off = (int64_t)kvh * p.block_size * D;
    k_base = reinterpret_cast<const T*>(p.key) + head_off;
    v_base = reinterpret_cast<const T*>(p.value) + head_off;
  } else {
    const int64_t head_off = (int64_t)b * p.kv_stride_b + (int64_t)kvh * p.kv_stride_h;
    k_base = reinterpret_cast<const T*>(p.key) + head_off;
    v_base = reinterpret_cast<const T*>(p.value) + head_off;
  }
  const int32_t* table_row = paged ? p.page_table + (int64_t)b * p.table_stride : nullptr;

  const uint32_t warp_smem_u32 = smem_u32(smem_raw + warp * Cfg::kWarpSmem);
  volatile int* stage_flags = reinterpret_cast<volatile int*>(smem_raw + kMmaWarps * Cfg::kWarpSmem + warp * 16);

  // element offset of token t relative to k_base / v_base, or -1 when the token has no storage (hole in the table)
  auto token_offset = [&](uint32_t t) -> int64_t {
    if (!paged) return ring_len > 0 ? (int64_t)(t % (uint32_t)ring_len) * D : (int64_t)t * p.kv_stride_t;
    const uint32_t blk = block_shift >= 0 ? (t >> block_shift) : (t / block_size);
    const uint32_t in_page = t - blk * block_size;
    const int32_t pid = table_row[blk];
    if (pid < 0 || pid >= p.num_pages) return -1;
    return (int64_t)pid * p.page_stride + (int64_t)(in_page * D);
  };

  // lane-constant parts of the copy pattern: copy i moves chunk `col` of tile row (i * kRowsPerCopy + row0)
  const int row0 = lane / Cfg::kChunksPerRow;
  const int col = lane % Cfg::kChunksPerRow;

  // Issue the async copies of tile `tile` (tokens [ts, ts+16)) into stage `stage`; rows without a token are zero-filled.
  auto issue_tile = [&](int tile, int stage) {
    const int ts = t0 + tile * kTileTokens;
    const int valid = min(kTileTokens, t1 - ts);
    const uint32_t k_dst = warp_smem_u32 + stage * 2 * Cfg::kTileBytes;
    const uint32_t v_dst = k_dst + Cfg::kTileBytes;
    if (tile_contiguous) {
      const int64_t tile_off = token_offset((uint32_t)ts);
      if (lane == 0) stage_flags[stage] = tile_off >= 0 ? valid : 0;
      const T* k_src = k_base + (tile_off >= 0 ? tile_off : 0) + col * 8;
      const T* v_src = v_base + (tile_off >= 0 ? tile_off : 0) + col * 8;
#pragma unroll
      for (int i = 0; i < Cfg::kCopiesPerLane; ++i) {
        const int row = i * Cfg::kRowsPerCopy + row0;
        const bool ok = (row < valid) && (tile_off >= 0);
        const uint32_t dst = swizzled_offset(row, col, Cfg::kRowBytes);
        cp_async16(k_dst + dst, k_src + (ok ? row * D : 0), ok ? 16 : 0);
        cp_async16(v_dst + dst, v_src + (ok ? row * D : 0), ok ? 16 : 0);
      }
    } else {
      if (lane == 0) stage_flags[stage] = -1;  // rows are validated one by one at compute time
#pragma unroll
      for (int i = 0; i < Cfg::kCopiesPerLane; ++i) {
        const int row = i * Cfg::kRowsPerCopy + row0;
        const int64_t off = row < valid ? token_offset((uint32_t)(ts + row)) : -1;
        const bool ok = off >= 0;
        const uint32_t dst = swizzled_offset(row, col, Cfg::kRowBytes);
        cp_async16(k_dst + dst, k_base + (ok ? off : 0) + col * 8, ok ? 16 : 0);
        cp_async16(v_dst + dst, v_base + (ok ? off : 0) + col * 8, ok ? 16 : 0);
      }
    }
  };

  // ---- per-warp online softmax state (two head columns per lane: 2tig, 2tig+1) ---------------------------------------
  const float sm_scale = p.scaling * 1.4426950408889634f;  // scores are kept in log2 units
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  float o_acc[Cfg::kSteps][4];
#pragma unroll
  for (int j = 0; j < Cfg::kSteps; ++j)
#pragma unroll
    for (int r = 0; r < 4; ++r) o_acc[j][r] = 0.0f;

  const int my_tiles = num_tiles > warp ? (num_tiles - warp + kMmaWarps - 1) / kMmaWarps : 0;
#pragma unroll
  for (int s = 0; s < Cfg::kStages - 1; ++s) {
    if (s < my_tiles) issue_tile(warp + s * kMmaWarps, s);
    cp_async_commit();
  }

  // ldmatrix lane addressing: matrix id mi = lane / 8, row-in-matrix = lane % 8
  const int mi = lane >> 3;
  const int k_row = (lane & 7) + 8 * (mi & 1);   // K (non-transposed): matrices ordered (rows 0-7 | 8-15) x (chunk 2s | 2s+1)
  const int k_chunk_sel = mi >> 1;
  const int v_row = (lane & 7) + 8 * (mi >> 1);  // V (transposed): matrices ordered (chunk 2j | 2j+1) x (rows 0-7 | 8-15)
  const int v_chunk_sel = mi & 1;
  uint32_t k_lds[Cfg::kSteps], v_lds[Cfg::kSteps];  // per-step shared offsets inside a tile (lane constants)
#pragma unroll
  for (int ks = 0; ks < Cfg::kSteps; ++ks) {
    k_lds[ks] = swizzled_offset(k_row, 2 * ks + k_chunk_sel, Cfg::kRowBytes);
    v_lds[ks] = swizzled_offset(v_row, 2 * ks + v_chunk_sel, Cfg::kRowBytes);
  }

  for (int n = 0; n < my_tiles; ++n) {
    __syncwarp();
    const int next = n + Cfg::kStages - 1;
    if (next < my_tiles) issue_tile(warp + next * kMmaWarps, next % Cfg::kStages);
    cp_async_commit();
    cp_async_wait<Cfg::kStages - 1>();
    __syncwarp();

    const int stage = n % Cfg::kStages;
    const uint32_t k_src = warp_smem_u32 + stage * 2 * Cfg::kTileBytes;
    const uint32_t v_src = k_src + Cfg::kTileBytes;
    const int flag = stage_flags[stage];

    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float s_odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // two accumulator chains halve the dependent-MMA latency
#pragma unroll
    for (int ks = 0; ks < Cfg::kSteps; ks += 2) {
      uint32_t a[4], a2[4];
      ldmatrix_x4(a, k_src + k_lds[ks]);
      ldmatrix_x4(a2, k_src + k_lds[ks + 1]);
      mma_m16n8k16<T>(s, a, qf[ks][0], qf[ks][1]);
      mma_m16n8k16<T>(s_odd, a2, qf[ks + 1][0], qf[ks + 1][1]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) s[r] = (s[r] + s_odd[r]) * sm_scale;

    if (flag != kTileTokens) {  // partial or hole tile: tokens without storage score -inf
      bool ok_lo, ok_hi;
      if (flag >= 0) {
        ok_lo = gid < flag;
        ok_hi = gid + 8 < flag;
      } else {
        const int ts = t0 + (warp + n * kMmaWarps) * kTileTokens;
        const int valid = min(kTileTokens, t1 - ts);
        ok_lo = gid < valid && token_offset((uint32_t)(ts + gid)) >= 0;
        ok_hi = gid + 8 < valid && token_offset((uint32_t)(ts + gid + 8)) >= 0;
      }
      if (!ok_lo) s[0] = s[1] = -INFINITY;
      if (!ok_hi) s[2] = s[3] = -INFINITY;
    }

    float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
    for (int d = 4; d <= 16; d <<= 1) {
      mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], d));
      mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], d));
    }
    const float m_new[2] = {fmaxf(m_run[0], mx[0]), fmaxf(m_run[1], mx[1])};
    const bool grew = (m_new[0] > m_run[0]) || (m_new[1] > m_run[1]);
    const float m_safe[2] = {m_new[0] == -INFINITY ? 0.0f : m_new[0], m_new[1] == -INFINITY ? 0.0f : m_new[1]};
    if (__any_sync(0xffffffffu, grew)) {
      const float a0 = exp2f(m_run[0] - m_safe[0]);
      const float a1 = exp2f(m_run[1] - m_safe[1]);
      l_run[0] *= a0;
      l_run[1] *= a1;
#pragma unroll
      for (int j = 0; j < Cfg::kSteps; ++j) {
        o_acc[j][0] *= a0;
        o_acc[j][1] *= a1;
        o_acc[j][2] *= a0;
        o_acc[j][3] *= a1;
      }
      m_run[0] = m_new[0];
      m_run[1] = m_new[1];
    }
    const float p0 = exp2f(s[0] - m_safe[0]);
    const float p1 = exp2f(s[1] - m_safe[1]);
    const float p2 = exp2f(s[2] - m_safe[0]);
    const float p3 = exp2f(s[3] - m_safe[1]);
    l_run[0] += p0 + p2;
    l_run[1] += p1 + p3;
    // P^T fragments: b0 = P[tok 2tig..+1][head gid], b1 = P[tok 2tig+8..+9][head gid]
    const uint32_t pb0 = movmatrix_trans(pack2<T>(p0, p1));
    const uint32_t pb1 = movmatrix_trans(pack2<T>(p2, p3));
#pragma unroll
    for (int j = 0; j < Cfg::kSteps; ++j) {
      uint32_t a[4];
      ldmatrix_x4_trans(a, v_src + v_lds[j]);
      mma_m16n8k16<T>(o_acc[j], a, pb0, pb1);
    }
  }
  cp_async_wait<0>();

  // ---- merge the four warps and write one partial per query head -----------------------------------------------------
#pragma unroll
  for (int d = 4; d <= 16; d <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], d);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], d);
  }
  __syncthreads();  // every warp is done with its pipeline buffers
  float* sm_m = reinterpret_cast<float*>(smem_raw);   // [warps][8]
  float* sm_l = sm_m + kMmaWarps * 8;                  // [warps][8]
  float* sm_o = sm_l + kMmaWarps * 8;                  // [warps][8][D + 4] (padded rows: conflict-free scatter)
  constexpr int kPad = D + 4;
  if (gid == 0) {
    sm_m[warp * 8 + 2 * tig] = m_run[0];
    sm_m[warp * 8 + 2 * tig + 1] = m_run[1];
    sm_l[warp * 8 + 2 * tig] = l_run[0];
    sm_l[warp * 8 + 2 * tig + 1] = l_run[1];
  }
#pragma unroll
  for (int j = 0; j < Cfg::kSteps; ++j) {
    float* base = sm_o + (warp * 8) * kPad;
    base[(2 * tig) * kPad + 16 * j + gid] = o_acc[j][0];
    base[(2 * tig + 1) * kPad + 16 * j + gid] = o_acc[j][1];
    base[(2 * tig) * kPad + 16 * j + gid + 8] = o_acc[j][2];
    base[(2 * tig + 1) * kPad + 16 * j + gid + 8] = o_acc[j][3];
  }
  __syncthreads();
  const int64_t part = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity + slot;
  float* stats_out = p.stats + part * 2;
  float* values_out = p.values + part * D;
  for (int item = threadIdx.x; item < g_count * D; item += kMmaThreads) {
    const int g = item / D;
    const int d = item % D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) m_all = fmaxf(m_all, sm_m[w * 8 + g]);
    const float m_ref = m_all == -INFINITY ? 0.0f : m_all;
    float l_all = 0.0f, o_all = 0.0f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float wgt = exp2f(sm_m[w * 8 + g] - m_ref);
      l_all += sm_l[w * 8 + g] * wgt;
      o_all += sm_o[(w * 8 + g) * kPad + d] * wgt;
    }
    values_out[(int64_t)g * p.chunk_capacity * D + d] = o_all;
    if (d == 0) {
      // the combine pass works in natural-log units
      stats_out[(int64_t)g * p.chunk_capacity * 2 + 0] = m_all * 0.6931471805599453f;
      stats_out[(int64_t)g * p.chunk_capacity * 2 + 1] = l_all;
    }
  }
  if (p.fused.counters != nullptr) {
    const int64_t head0 = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity;
    __syncthreads();  // the epilogue buffers above are dead; reuse shared memory for the merge weights
    fused_combine_tail<T, D, kMmaThreads>(p.fused, b, hq0, g_count, active_chunks, p.chunk_capacity,
                                          p.stats + head0 * 2, p.values + head0 * D,
                                          reinterpret_cast<float*>(smem_raw), counter_index);
  }
}

}  // namespace anna
