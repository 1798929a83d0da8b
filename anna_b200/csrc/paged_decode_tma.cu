// Paged single-token GQA decode for 16-bit K/V with TMA tile loads (sm_100a).
//
// The page pools are described to the TMA unit as 2-D tensors [pages * kv_heads * page_size rows, head_dim columns];
// a 16-token tile of one kv head is head_dim / 64 boxes of 16 rows x 128 bytes, written to shared memory with the
// hardware 128-byte swizzle, which is exactly the bank-conflict-free layout ldmatrix wants.  One lane per warp issues
// the copies of a tile (cp.async.bulk.tensor.2d, completion counted in bytes on an mbarrier) several tiles ahead of the
// warp's own consumption, so no thread computes per-16-byte addresses and no register is spent on data in flight:
//
//   page pool --TMA, 128B swizzle--> shared ring (kStages tiles per warp) --ldmatrix--> mma.sync m16n8k16
//   S[16 tok x 8 heads] = K_tile . Q^T,  online softmax in fp32,  O^T[D x 8 heads] += V_tile^T . P^T
//
// Work is dealt by the even-share schedule (balanced_schedule.cuh) with the warp as the unit; the partials of a stream
// are merged by the warp whose partial arrives last.  Every mbarrier wait is bounded: on expiry the warp records a fault,
// stops consuming and the kernel still runs to completion.
#include <cuda.h>  // CUtensorMap and its enums; the encoder is looked up at run time, nothing links against libcuda

#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <vector>

#include "balanced_schedule.cuh"
#include "decode_core.cuh"
#include "decode_params.cuh"
#include "mbarrier_utils.cuh"
#include "mma_utils.cuh"
#include "tq_decode_params.cuh"

#ifndef ANNA_TMA_STAGES
#define ANNA_TMA_STAGES 2
#endif
#ifndef ANNA_TMA_WARPS
#define ANNA_TMA_WARPS 4
#endif

namespace anna {

constexpr int kTmaWarps = ANNA_TMA_WARPS;
constexpr int kTmaThreads = kTmaWarps * 32;
constexpr int kTmaTile = 16;          // tokens per tile (the M of the MMA)
constexpr int kBoxCols = 64;          // 16-bit elements per box row = 128 bytes = the swizzle span
constexpr int kBoxBytes = kTmaTile * 128;

__device__ int32_t g_tma_decode_faults;  // bumped when a bounded mbarrier wait expires


template <int D>
struct TmaCfg {
  static constexpr int kSteps = D / 16;
  static constexpr int kBoxes = D / kBoxCols;             // boxes per K (or V) tile
  static constexpr int kTileBytes = kBoxes * kBoxBytes;   // K (or V) tile
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kStages = ANNA_TMA_STAGES;
  static constexpr int kWarpBytes = kStages * kStageBytes;
  static constexpr int kRingBytes = kTmaWarps * kWarpBytes;
  static constexpr int kBarrierBytes = kTmaWarps * kStages * 8;
  static constexpr int kFlagBytes = kTmaWarps * kStages * 8;
  static constexpr int kSmemBytes = kRingBytes + kBarrierBytes + kFlagBytes + 1024;  // + slack to align the ring
  // resident CTAs per SM the launch bound asks for (registers: 65536 / (threads * blocks))
  static constexpr int kMinBlocks = (200 * 1024) / kSmemBytes >= 3 ? 3 : ((200 * 1024) / kSmemBytes >= 2 ? 2 : 1);
  static_assert(D % kBoxCols == 0, "head_dim must be a multiple of 64");
};

// ---- tiled TMA load (mbarrier helpers: mbarrier_utils.cuh) --------------------------------------------------------------
// One box: columns [x, x + 64) of rows [y, y + 16) -> shared `dst` (1024-byte aligned), completion bytes on `bar`.
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Merge of the split-K partials of one stream by a single warp (the one whose partial arrived last).
// stats / values point at slot 0 of query head hq0.  Each lane owns D / 32 consecutive output elements.
// The merge sits on the critical path at the end of the kernel and is pure L2 latency, so it is arranged as two
// round trips: lane c fetches the (max, sum) of partial c for all heads at once and the weights are formed with
// warp reductions; then the value rows are fetched with all heads of two partials in flight together.
template <typename T, int D>
__device__ __forceinline__ void warp_merge_stream(const FusedCombine& fc, int b, int hq0, int g_count, int partials,
                                                  int chunk_capacity, const float* stats, const float* values) {
  constexpr int E = D / 32;
  using Vec = typename std::conditional<E == 2, float2, float4>::type;
  constexpr int kVecs = E == 2 ? 1 : E / 4;
  const int lane = threadIdx.x & 31;
  const int64_t head_stride = (int64_t)chunk_capacity * D;
  auto store_head = [&](int g, const float (&acc)[E], float inv) {
    T* out = reinterpret_cast<T*>(fc.out) + (int64_t)b * fc.out_stride_b + (int64_t)(hq0 + g) * fc.out_stride_h +
             lane * E;
    const T* gate = fc.gate ? reinterpret_cast<const T*>(fc.gate) + (int64_t)b * fc.gate_stride_b +
                                  (int64_t)(hq0 + g) * fc.gate_stride_h + lane * E
                            : nullptr;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      float v = acc[e] * inv;
      if (gate) v *= sigmoidf_fast(ElemTraits<T>::to_float(gate[e]));
      out[e] = ElemTraits<T>::from_float(v);
    }
  };
  auto accumulate = [&](float (&acc)[E], const Vec (&v)[kVecs], float w) {
    if constexpr (E == 2) {
      acc[0] = fmaf(v[0].x, w, acc[0]);
      acc[1] = fmaf(v[0].y, w, acc[1]);
    } else {
#pragma unroll
      for (int k = 0; k < kVecs; ++k) {
        acc[4 * k + 0] = fmaf(v[k].x, w, acc[4 * k + 0]);
        acc[4 * k + 1] = fmaf(v[k].y, w, acc[4 * k + 1]);
        acc[4 * k + 2] = fmaf(v[k].z, w, acc[4 * k + 2]);
        acc[4 * k + 3] = fmaf(v[k].w, w, acc[4 * k + 3]);
      }
    }
  };

  if (partials <= 32) {
    // round trip 1: lane c holds the weight of partial c for every head
    float w[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float2 ml = make_float2(-INFINITY, 0.0f);
      if (g < g_count && lane < partials)
        ml = __ldcg(reinterpret_cast<const float2*>(stats + ((int64_t)g * chunk_capacity + lane) * 2));
      w[g] = ml.x;
      float m = ml.x;
#pragma unroll
      for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
      const float e = __expf(w[g] - (m == -INFINITY ? 0.0f : m));  // exp(-inf) = 0 for lanes without a partial
      float den = ml.y * e;
#pragma unroll
      for (int d = 16; d >= 1; d >>= 1) den += __shfl_xor_sync(0xffffffffu, den, d);
      w[g] = den > 0.0f ? e / den : 0.0f;
    }
    // round trip 2..: value rows, all heads of two partials per batch
    float acc[8][E];
#pragma unroll
    for (int g = 0; g < 8; ++g)
#pragma unroll
      for (int e = 0; e < E; ++e) acc[g][e] = 0.0f;
    const float* vals = values + lane * E;
    constexpr bool kPair = E <= 4;  // wide rows: one partial per batch keeps the loads in registers
#pragma unroll 1
    for (int c = 0; c < partials; c += kPair ? 2 : 1) {
      Vec v0[8][kVecs], v1[kPair ? 8 : 1][kVecs];
      const bool two = kPair && c + 1 < partials;
#pragma unroll
      for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int k = 0; k < kVecs; ++k) {
          if (g < g_count) {
            v0[g][k] = __ldcg(reinterpret_cast<const Vec*>(vals + g * head_stride + (int64_t)c * D) + k);
            if constexpr (kPair)
              if (two) v1[g][k] = __ldcg(reinterpret_cast<const Vec*>(vals + g * head_stride + (int64_t)(c + 1) * D) + k);
          }
        }
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float w0 = __shfl_sync(0xffffffffu, w[g], c);
        const float w1 = __shfl_sync(0xffffffffu, w[g], (c + 1) & 31);
        if (g < g_count) {
          accumulate(acc[g], v0[g], w0);
          if constexpr (kPair)
            if (two) accumulate(acc[g], v1[g], w1);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < 8; ++g)
      if (g < g_count) store_head(g, acc[g], 1.0f);
    return;
  }

  // many partials per stream (a long row among short ones): head by head
  for (int g = 0; g < g_count; ++g) {
    const float* st = stats + (int64_t)g * chunk_capacity * 2;
    const float* vals = values + g * head_stride + lane * E;
    float m = -INFINITY;
    for (int c = lane; c < partials; c += 32) m = fmaxf(m, __ldcg(st + 2 * c));
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float m_ref = m == -INFINITY ? 0.0f : m;
    float den = 0.0f;
    float acc[E];
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = 0.0f;
#pragma unroll 4
    for (int c = 0; c < partials; ++c) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(st + 2 * c));
      const float w = __expf(ml.x - m_ref);
      den = fmaf(ml.y, w, den);
      Vec v[kVecs];
#pragma unroll
      for (int k = 0; k < kVecs; ++k) v[k] = __ldcg(reinterpret_cast<const Vec*>(vals + (int64_t)c * D) + k);
      accumulate(acc, v, w);
    }
    store_head(g, acc, den > 0.0f ? 1.0f / den : 0.0f);
  }
}

// One stream a warp works on: a (row, kv head, group of <= 8 query heads) and where its partial goes.
struct StreamRef {
  int b;         // row
  int stream;    // stream inside the row
  int n;         // tiles of the stream
  int first;     // line position of its first tile
};

// The kernel.  Every warp is a work unit of its own; the CTA is only a container (no CTA barrier after the prologue).
//
// Static part: the even-share arithmetic (balanced_schedule.cuh) gives unit u the line range [u * share, (u + 1) * share)
// and with it the list of streams the unit is attached to, its partial slot in each of them and the number of partials
// each stream will receive.  Unit numbers are a fixed scramble of (warp, CTA), so the units attached to one stream sit
// on SMs far apart.
// Dynamic part: the tiles of a stream are not split in advance.  Each attached warp claims the next tile of the stream
// from a per-stream cursor (one atomicAdd per tile, issued one tile ahead so that its latency is hidden) until the
// stream is exhausted -- or, on every stream of its list but the last, until it has taken as many tiles as its static
// overlap -- and then moves on.  SMs do not all reach the same memory bandwidth (measured spread about +-10 %); with
// claiming, a warp on a fast SM simply takes more tiles of the stream it shares with slower ones.
// Per warp: lane 0 starts the TMA copies of a claimed tile into the next ring stage (kept kStages ahead, across stream
// boundaries, so the copy pipeline never drains); all lanes consume tiles in the same order.  After the last tile of a
// stream the warp publishes its partial (an empty one if it got no tile), and the warp whose partial arrives last
// merges the stream and puts both counters back to zero.
template <typename T, int D>
__global__ void __launch_bounds__(kTmaThreads, TmaCfg<D>::kMinBlocks)
paged_decode_tma_kernel(const DenseDecodeParams p, const int batch, const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map) {
  using Cfg = TmaCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_unaligned[];
  __shared__ int s_prefix[kBalancedMaxRows + 1];
  // the swizzle pattern is a function of the shared address: every box must start on a 1024-byte boundary
  uint8_t* smem_raw = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2;
  const int tig = lane & 3;
  if (threadIdx.x == 0) {
    const uint32_t bars = smem_u32(smem_raw + Cfg::kRingBytes);
    for (int i = 0; i < kTmaWarps * Cfg::kStages; ++i) mbar_init(bars + i * 8, 1);
    mbar_init_fence();
  }
  const int group_tiles = (p.groups + 7) / 8;
  const int streams_per_row = p.kv_heads * group_tiles;
  const int max_tiles = balanced_scan<kTmaThreads>(p.visible_lengths, p.max_len, batch, streams_per_row, s_prefix);
  const int total = s_prefix[batch];  // (the scan ends with a CTA barrier: the mbarriers are initialised for everyone)

  // rows without a visible key have no tile: their zero outputs are dealt round-robin over the CTAs
  for (int b = blockIdx.x; b < batch; b += gridDim.x) {
    if (s_prefix[b + 1] != s_prefix[b]) continue;
    for (int stream = 0; stream < streams_per_row; ++stream) {
      const int g0 = (stream % group_tiles) * 8;
      fused_write_zero_row<T, D, kTmaThreads>(p.fused, b, (stream / group_tiles) * p.groups + g0, min(8, p.groups - g0));
    }
  }
  if (total == 0) return;
  // logical unit of this warp: a fixed scramble of (warp, CTA), so that neighbours in the line sit on distant SMs
  const int units = (int)gridDim.x * kTmaWarps;
  int scramble = 61;
  for (;; scramble += 2) {
    int a = units, c = scramble;
    while (c != 0) { const int r = a % c; a = c; c = r; }
    if (a == 1) break;  // coprime with the number of units: the map is a permutation
  }
  const int unit = (int)(((int64_t)(warp * (int)gridDim.x + (int)blockIdx.x) * scramble) % units);
  const int share = balanced_share(total, units, max_tiles, p.chunk_capacity, 1);
  const int begin = (int)min((int64_t)unit * share, (int64_t)total);
  const int end = (int)min((int64_t)begin + share, (int64_t)total);
  if (begin >= end) return;

  const uint32_t ring_u32 = smem_u32(smem_raw + warp * Cfg::kWarpBytes);
  uint8_t* ring_ptr = smem_raw + warp * Cfg::kWarpBytes;
  const uint32_t bars_u32 = smem_u32(smem_raw + Cfg::kRingBytes + warp * Cfg::kStages * 8);
  // per stage: which stream of this warp's list the tile belongs to, and how many of its 16 rows are tokens
  volatile int2* stage_meta = reinterpret_cast<volatile int2*>(smem_raw + Cfg::kRingBytes + Cfg::kBarrierBytes) +
                              warp * Cfg::kStages;
  const int block_shift = p.block_shift;
  const uint32_t block_size = (uint32_t)p.block_size;
  int32_t* arrivals = p.fused.counters;                                    // [batch * streams_per_row]
  int32_t* cursors = p.fused.counters + (int64_t)batch * streams_per_row;  // [batch * streams_per_row]

  // Walks the streams that overlap [begin, end) in line order.
  auto stream_at = [&](int pos) -> StreamRef {
    TileCursor c;
    c.seek(s_prefix, batch, streams_per_row, pos);
    return StreamRef{c.b, c.stream, c.n, c.stream_first()};
  };
  auto next_stream = [&](const StreamRef& s) -> StreamRef {  // only called when s.first + s.n < end
    return stream_at(s.first + s.n);
  };

  // ---- producer state (all warp-uniform) ----------------------------------------------------------------------------------
  StreamRef prod = stream_at(begin);
  int prod_index = 0;      // position of `prod` in this warp's list
  bool prod_done = false;
  uint32_t issued = 0, consumed = 0;
  int pending = 0;         // lane 0: tile claimed ahead of time from prod's cursor
  int taken = 0;           // tiles this warp started from prod
  // A warp may take more than its static overlap only from the last stream of its list: it has to leave the earlier
  // ones on time, or every later stream would get its shared warp late.
  auto quota = [&]() -> int {
    return prod.first + prod.n >= end ? prod.n : min(end, prod.first + prod.n) - max(begin, prod.first);
  };
  auto claim = [&]() {
    if (taken >= quota()) {
      pending = prod.n;  // behaves like an exhausted stream
    } else if (lane == 0) {
      pending = atomicAdd(cursors + (int64_t)prod.b * streams_per_row + prod.stream, 1);
    }
  };
  claim();
  // Starts at most one more tile; afterwards either a tile was issued, the ring is full, or the list is exhausted.
  auto produce = [&]() {
    if (prod_done || issued - consumed >= (uint32_t)Cfg::kStages) return;
    for (;;) {
      const int tile = __shfl_sync(0xffffffffu, pending, 0);
      if (tile < prod.n) {
        const uint32_t stage = issued % Cfg::kStages;
        ++issued;
        ++taken;
        if (lane == 0) {
          const uint32_t ts = (uint32_t)tile * kTmaTile;
          const uint32_t blk = block_shift >= 0 ? (ts >> block_shift) : (ts / block_size);
          const uint32_t in_page = ts - blk * block_size;
          const int32_t pid = p.page_table[(int64_t)prod.b * p.table_stride + blk];
          const uint32_t bar = bars_u32 + stage * 8;
          if (pid < 0 || pid >= p.num_pages) {  // hole in the block table: nothing to copy, the phase completes at once
            stage_meta[stage].x = prod_index;
            stage_meta[stage].y = 0;
            mbar_arrive(bar);
          } else {
            int64_t len = p.visible_lengths ? p.visible_lengths[prod.b] : p.max_len;
            len = max((int64_t)0, min(len, p.max_len));
            stage_meta[stage].x = prod_index;
            stage_meta[stage].y = (int)min((int64_t)kTmaTile, len - (int64_t)ts);
            const int kvh = prod.stream / group_tiles;
            const int y = (int)(((int64_t)pid * p.kv_heads + kvh) * block_size + in_page);
            const uint32_t dst = ring_u32 + stage * Cfg::kStageBytes;
            mbar_expect_tx(bar, Cfg::kStageBytes);
#pragma unroll
            for (int h = 0; h < Cfg::kBoxes; ++h) {
              tma_load_box(dst + h * kBoxBytes, &k_map, h * kBoxCols, y, bar);
              tma_load_box(dst + Cfg::kTileBytes + h * kBoxBytes, &v_map, h * kBoxCols, y, bar);
            }
          }
        }
        claim();  // the next tile of the same stream, needed one call from now
        return;
      }
      // this stream has no tile left: move down the list
      if (prod.first + prod.n >= end) {
        prod_done = true;
        return;
      }
      prod = next_stream(prod);
      ++prod_index;
      taken = 0;
      claim();
    }
  };
#pragma unroll 1
  for (int s = 0; s < Cfg::kStages; ++s) produce();

  // ldmatrix lane addressing inside a swizzled box: row r, 16-byte chunk c -> r * 128 + ((c ^ (r & 7)) << 4)
  const int mi = lane >> 3;
  const int k_row = (lane & 7) + 8 * (mi & 1);   // K: matrices ordered (rows 0-7 | 8-15) x (chunk 2s | 2s+1)
  const int k_sel = mi >> 1;
  const int v_row = (lane & 7) + 8 * (mi >> 1);  // V^T: matrices ordered (chunk 2j | 2j+1) x (rows 0-7 | 8-15)
  const int v_sel = mi & 1;
  uint32_t k_lds[Cfg::kSteps], v_lds[Cfg::kSteps];
#pragma unroll
  for (int s = 0; s < Cfg::kSteps; ++s) {
    const int kc = 2 * s + k_sel, vc = 2 * s + v_sel;  // chunk index inside the token row
    k_lds[s] = (kc >> 3) * kBoxBytes + k_row * 128 + (((kc & 7) ^ (k_row & 7)) << 4);
    v_lds[s] = Cfg::kTileBytes + (vc >> 3) * kBoxBytes + v_row * 128 + (((vc & 7) ^ (v_row & 7)) << 4);
  }
  const float sm_scale = p.scaling * 1.4426950408889634f;  // scores are kept in log2 units

  // ---- consumer: the streams of the list, one after the other ---------------------------------------------------------------
  StreamRef cons = stream_at(begin);
  bool broken = false;
  for (int cons_index = 0;; ++cons_index) {
    const int b = cons.b;
    const int kvh = cons.stream / group_tiles;
    const int g0 = (cons.stream % group_tiles) * 8;
    const int g_count = min(8, p.groups - g0);
    const int hq0 = kvh * p.groups + g0;
    const int first_unit = cons.first / share;
    const int slot = unit - first_unit;
    const int partials = (cons.first + cons.n - 1) / share - first_unit + 1;

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
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.0f, 0.0f};
    float o_acc[Cfg::kSteps][4];
#pragma unroll
    for (int j = 0; j < Cfg::kSteps; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) o_acc[j][r] = 0.0f;

#pragma unroll 1
    while (!broken) {
      produce();
      __syncwarp();  // lane 0's stage bookkeeping is visible to the other lanes
      if (consumed == issued) break;  // nothing in flight: the producer is past this stream
      const uint32_t stage = consumed % Cfg::kStages;
      if (stage_meta[stage].x != cons_index) break;  // the oldest tile in flight belongs to a later stream
      const uint32_t parity = (consumed / Cfg::kStages) & 1u;
      ++consumed;
      if (!mbar_wait(bars_u32 + stage * 8, parity)) {
        if (lane == 0) atomicAdd(&g_tma_decode_faults, 1);
        broken = true;
        break;
      }
      const int flag = stage_meta[stage].y;
      const uint32_t src = ring_u32 + stage * Cfg::kStageBytes;
      if (flag != kTmaTile) {
        if (flag == 0) {  // hole: no token of this tile exists
          __syncwarp();
          continue;
        }
        // last, partial tile of the row: rows past the end hold stale bytes; clear their V so that 0 * stale is 0
        for (int item = lane; item < (kTmaTile - flag) * (D / 8); item += 32) {
          const int row = flag + item / (D / 8);
          const int c = item % (D / 8);
          const uint32_t off = Cfg::kTileBytes + (c >> 3) * kBoxBytes + row * 128 + (((c & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(ring_ptr + stage * Cfg::kStageBytes + off) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // order these stores before the next TMA write
        __syncwarp();
      }

      float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      float s_odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // two accumulator chains halve the dependent-MMA latency
#pragma unroll
      for (int ks = 0; ks < Cfg::kSteps; ks += 2) {
        uint32_t a[4], a2[4];
        ldmatrix_x4(a, src + k_lds[ks]);
        ldmatrix_x4(a2, src + k_lds[ks + 1]);
        mma_m16n8k16<T>(s, a, qf[ks][0], qf[ks][1]);
        mma_m16n8k16<T>(s_odd, a2, qf[ks + 1][0], qf[ks + 1][1]);
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) s[r] = (s[r] + s_odd[r]) * sm_scale;
      if (flag != kTmaTile) {
        if (gid >= flag) s[0] = s[1] = -INFINITY;
        if (gid + 8 >= flag) s[2] = s[3] = -INFINITY;
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
      const uint32_t pb0 = movmatrix_trans(pack2<T>(p0, p1));
      const uint32_t pb1 = movmatrix_trans(pack2<T>(p2, p3));
#pragma unroll
      for (int j = 0; j < Cfg::kSteps; ++j) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, src + v_lds[j]);
        mma_m16n8k16<T>(o_acc[j], a, pb0, pb1);
      }
      __syncwarp();  // every lane is done with this stage before lane 0 re-arms it
    }

    // ---- publish this warp's partial of the stream: (max, sum) and O for up to 8 heads ------------------------------------
#pragma unroll
    for (int d = 4; d <= 16; d <<= 1) {
      l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], d);
      l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], d);
    }
    const int64_t head0 = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity;
    float* stats0 = p.stats + head0 * 2;
    float* values0 = p.values + head0 * D;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int g = 2 * tig + r;
      if (g < g_count) {
        float* vout = values0 + ((int64_t)g * p.chunk_capacity + slot) * D;
#pragma unroll
        for (int j = 0; j < Cfg::kSteps; ++j) {
          vout[16 * j + gid] = o_acc[j][r];
          vout[16 * j + gid + 8] = o_acc[j][r + 2];
        }
        if (gid == 0) {
          float2 ml;
          ml.x = m_run[r] * 0.6931471805599453f;  // natural-log units
          ml.y = l_run[r];
          *reinterpret_cast<float2*>(stats0 + ((int64_t)g * p.chunk_capacity + slot) * 2) = ml;
        }
      }
    }
    // last arriver merges: nobody waits for anybody
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      const int64_t stream_index = (int64_t)b * streams_per_row + cons.stream;
      const int prev = atomicAdd(arrivals + stream_index, 1);
      last = prev == partials - 1;
      if (last) {  // every attached warp is done claiming: the caller's buffer goes back to all-zero
        arrivals[stream_index] = 0;
        cursors[stream_index] = 0;
      }
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      __threadfence();
      warp_merge_stream<T, D>(p.fused, b, hq0, g_count, partials, p.chunk_capacity, stats0, values0);
    }
    if (broken || cons.first + cons.n >= end) break;
    cons = next_stream(cons);
  }
  if (broken) {
    // copies that were started but not awaited: one more bounded chance to land before the CTA's memory is released
    while (consumed < issued) {
      (void)mbar_wait(bars_u32 + (consumed % Cfg::kStages) * 8, (consumed / Cfg::kStages) & 1u);
      ++consumed;
    }
  }
}

// ---- host side: tensor maps -----------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

struct PoolMapKey {
  int device;
  const void* base;
  uint64_t rows;
  int dim;
};
struct PoolMapEntry {
  PoolMapKey key;
  CUtensorMap map;
};

// Tensor map of one page pool viewed as [rows, dim] 16-bit elements, box 64 x 16, 128-byte swizzle (cached).
static bool pool_tensor_map(const void* base, uint64_t rows, int dim, CUtensorMap* out) {
  static std::mutex lock;
  static std::vector<PoolMapEntry> cache;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return false;
  std::lock_guard<std::mutex> guard(lock);
  for (const PoolMapEntry& e : cache)
    if (e.key.device == device && e.key.base == base && e.key.rows == rows && e.key.dim == dim) {
      *out = e.map;
      return true;
    }
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  PoolMapEntry entry{{device, base, rows, dim}, {}};
  const cuuint64_t global_dim[2] = {(cuuint64_t)dim, (cuuint64_t)rows};
  const cuuint64_t global_stride[1] = {(cuuint64_t)dim * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBoxCols, (cuuint32_t)kTmaTile};
  const cuuint32_t elem_stride[2] = {1, 1};
  const CUresult rc = encode(&entry.map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), global_dim,
                             global_stride, box, elem_stride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return false;
  if (cache.size() >= 64) cache.erase(cache.begin());
  cache.push_back(entry);
  *out = entry.map;
  return true;
}

template <typename T, int D>
static int launch_tma(const DenseDecodeParams& p, int batch, const CUtensorMap& k_map, const CUtensorMap& v_map,
                      cudaStream_t stream) {
  using Cfg = TmaCfg<D>;
  auto kernel = paged_decode_tma_kernel<T, D>;
  static int resident_ctas[64] = {};  // per device: CTAs of this kernel that fit the whole GPU at once
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  int ctas = (device >= 0 && device < 64) ? resident_ctas[device] : 0;
  if (ctas == 0) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    int sms = 0, per_sm = 0;
    ANNA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    ANNA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kTmaThreads, Cfg::kSmemBytes));
    ctas = sms * (per_sm > 0 ? per_sm : 1);
    if (device >= 0 && device < 64) resident_ctas[device] = ctas;
  }
  kernel<<<(unsigned)ctas, kTmaThreads, Cfg::kSmemBytes, stream>>>(p, batch, k_map, v_map);
  return check_launch("paged_decode_tma_kernel");
}

// ANNA_OK when the TMA kernel was launched, ANNA_ERR_UNSUPPORTED (no message) when this problem does not qualify and
// the caller should use the cp.async kernels instead.
int try_launch_paged_decode_tma(const DenseDecodeParams& p, int batch, int head_dim, int dtype, cudaStream_t stream) {
  // Opt-in: on the measured workloads (32-128 rows of 1-8 K tokens) this kernel reaches 5.1-6.0 TB/s where the
  // cp.async kernel with CTA-wide units reaches 5.8-6.1 TB/s, and it loses more on small batches.
  static const bool enabled = [] {
    const char* flag = std::getenv("ANNA_B200_PAGED_TMA");
    return flag != nullptr && flag[0] != '\0' && flag[0] != '0';
  }();
  if (!enabled || p.page_table == nullptr || p.fused.counters == nullptr) return ANNA_ERR_UNSUPPORTED;
  if (dtype != ANNA_DTYPE_F16 && dtype != ANNA_DTYPE_BF16) return ANNA_ERR_UNSUPPORTED;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return ANNA_ERR_UNSUPPORTED;
  if (p.block_size % kTmaTile != 0 || p.max_len >= (int64_t)1 << 31) return ANNA_ERR_UNSUPPORTED;
  if (!balanced_schedule_fits(batch, (int64_t)p.kv_heads * ((p.groups + 7) / 8), p.max_len, p.chunk_capacity))
    return ANNA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(p.key) & 15u) != 0 || (reinterpret_cast<uintptr_t>(p.value) & 15u) != 0)
    return ANNA_ERR_UNSUPPORTED;
  if (p.q_stride_b % 2 != 0 || p.q_stride_h % 2 != 0 || (reinterpret_cast<uintptr_t>(p.q) & 3u) != 0)
    return ANNA_ERR_UNSUPPORTED;
  // the merge reads partials as float2 / float4
  if ((reinterpret_cast<uintptr_t>(p.values) & 15u) != 0 || (reinterpret_cast<uintptr_t>(p.stats) & 7u) != 0)
    return ANNA_ERR_UNSUPPORTED;
  const uint64_t rows = (uint64_t)p.num_pages * (uint64_t)p.kv_heads * (uint64_t)p.block_size;
  if (rows >= ((uint64_t)1 << 31)) return ANNA_ERR_UNSUPPORTED;
  CUtensorMap k_map, v_map;
  if (!pool_tensor_map(p.key, rows, head_dim, &k_map) || !pool_tensor_map(p.value, rows, head_dim, &v_map))
    return ANNA_ERR_UNSUPPORTED;
  if (dtype == ANNA_DTYPE_BF16) {
    if (head_dim == 64) return launch_tma<__nv_bfloat16, 64>(p, batch, k_map, v_map, stream);
    if (head_dim == 128) return launch_tma<__nv_bfloat16, 128>(p, batch, k_map, v_map, stream);
    return launch_tma<__nv_bfloat16, 256>(p, batch, k_map, v_map, stream);
  }
  if (head_dim == 64) return launch_tma<__half, 64>(p, batch, k_map, v_map, stream);
  if (head_dim == 128) return launch_tma<__half, 128>(p, batch, k_map, v_map, stream);
  return launch_tma<__half, 256>(p, batch, k_map, v_map, stream);
}

}  // namespace anna

// ---- self-test of the bounded wait -------------------------------------------------------------------------------------------
namespace anna {
__global__ void wait_expiry_selftest_kernel(int32_t* result) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  __syncwarp();
  // nobody ever arrives on this barrier: the wait has to give up and say so
  const bool landed = mbar_wait(bar, 0u);
  if (threadIdx.x == 0) *result = landed ? 0 : 1;
}
}  // namespace anna

// Launches one warp that waits on an mbarrier nothing completes and reports whether the bounded wait gave up
// (*expired = 1) -- the path every copy wait of the library takes when its data does not arrive.  Takes about a second
// (the full wait budget), synchronises the stream, and leaves the context usable.  No counterpart in the reference.
extern "C" int anna_kv_selftest_wait_expiry(int* expired, anna_stream_t stream) {
  ANNA_REQUIRE(expired != nullptr, "anna_kv_selftest_wait_expiry: null output pointer");
  int32_t* flag = nullptr;
  ANNA_CUDA_CHECK(cudaMalloc(&flag, sizeof(int32_t)));
  cudaError_t err = cudaMemsetAsync(flag, 0xff, sizeof(int32_t), (cudaStream_t)stream);
  if (err == cudaSuccess) {
    anna::wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flag);
    err = cudaGetLastError();
  }
  int32_t value = -1;
  if (err == cudaSuccess) err = cudaMemcpyAsync(&value, flag, sizeof(value), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize((cudaStream_t)stream);
  cudaFree(flag);
  if (err != cudaSuccess) return anna::set_error(ANNA_ERR_CUDA, "wait-expiry self-test failed: %s", cudaGetErrorString(err));
  *expired = (int)value;
  return ANNA_OK;
}

// Number of bounded waits that expired in the kernels that stage tiles with the copy engine, on the current device, since the library was loaded
// (0 in a healthy run).  Synchronises the device.
extern "C" int anna_kv_device_faults(int* count) {
  ANNA_REQUIRE(count != nullptr, "anna_kv_device_faults: null output pointer");
  int32_t value = 0;
  ANNA_CUDA_CHECK(cudaMemcpyFromSymbol(&value, anna::g_tma_decode_faults, sizeof(value)));
  int packed = 0;
  const int rc = anna::tq_decode_mma_faults(&packed);
  if (rc != ANNA_OK) return rc;
  *count = (int)value + packed;
  return ANNA_OK;
}
