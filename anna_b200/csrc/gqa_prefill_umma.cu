// Multi-token (prefill / chunked-prefill) grouped-query attention on the 5th-generation tensor cores: tcgen05.mma with
// S, P and O in tensor memory.  head_dim 128 (first kernel), 256 and 64 (second kernel), 16-bit dtypes; same semantics as
// gqa_prefill.cu (grouped_query_attention, src/anna/model/ops.py:1552-1574, with the masks of ops.py:1840-1852 and
// :2008-2016).
//
// head_dim 128.  A CTA (one per SM) owns 256 rows = two query tiles of 128 rows: consecutive query positions of the (up
// to 16) query heads that share one KV head, so that a K / V tile fetched from L2 serves all of them (with 128 rows per
// K / V tile the copies from L2 bound an earlier version).  Eight softmax warps (thread t owns row t: lane t & 127 of
// query tile t >> 7) and one warp that issues every copy and every product from an elected lane; the parties meet on
// mbarriers only.  Per tile of 128 keys:
//   K / V tile --tiled TMA (two boxes of 64 values x 128 keys each, 128-byte swizzle, two stages each)--> shared memory;
//                                the rows of the one V tile that straddles the end of a row's keys are zeroed there (K
//                                needs nothing: its scores are masked)
//   S[128 x 128] = Q . K^T       per query tile 8 x tcgen05.mma kind::f16 (K = 16 each), Q and K K-major in shared
//                                memory, S in the tile's 128 score columns of tensor memory
//   softmax                      every thread reads its row of S into registers (tcgen05.ld): row maximum, exp2, row
//                                sum; P (16-bit pairs) overwrites the first 64 score columns (tcgen05.st).  The running
//                                maximum moves only when it would grow by more than 2^8, and only then is the row of O
//                                rescaled in tensor memory
//   O[128 x 128] += P . V        per query tile 8 x tcgen05.mma with P read from tensor memory (the A operand) and V
//                                MN-major in shared memory (the same byte arrangement as a K-major tile: only the
//                                descriptor's two strides swap roles), O in the tile's other 128 columns
// The tensor pipe sees P0.V | S0(next) | P1.V | S1(next): it runs in issue order, so S(next) overwrites P only after
// the product that reads it, and one query tile's products run during the other's softmax.
// Key tiles above the causal diagonal of the CTA's last row are never loaded.  Every wait is bounded: when one expires
// the CTA counts a fault, stops, and still frees its tensor memory.
#include "mma_utils.cuh"
#include "prefill_params.cuh"
#include "tma_utils.cuh"
#include "umma_utils.cuh"

#include <cstdlib>
#include <type_traits>

namespace anna {

__device__ int32_t g_prefill_umma_faults;

namespace {

constexpr int kUpQTiles = 2;      // query tiles (128 rows = one accumulator in tensor memory each) per CTA
constexpr int kUpRows = 128, kUpKeys = 128, kUpDim = 128;
constexpr int kUpCtaRows = kUpQTiles * kUpRows;
constexpr int kUpSoftmaxThreads = kUpCtaRows;       // one thread per query row (lane of tensor memory)
constexpr int kUpThreads = kUpSoftmaxThreads + 128;  // and a third group of four warps, one of which issues every copy and product
// Registers move between the groups of four warps: the issuing group keeps 136 per thread (its descriptors) and the softmax groups take
// 184, enough for a whole row of scores.  The CTA's pool is what it was launched with (384 threads x 168, the most the
// compiler may use at this CTA size); a group that asked for more than the pool holds would wait for ever.
constexpr int kUpLaunchRegs = 168, kUpIssuerRegs = 136, kUpSoftmaxRegs = 184;
static_assert(128 * kUpIssuerRegs + kUpSoftmaxThreads * kUpSoftmaxRegs <= kUpThreads * kUpLaunchRegs,
              "register split exceeds the CTA's pool");
static_assert(kUpLaunchRegs == (65536 / kUpThreads) / 8 * 8, "launch registers per thread");
// Q, K, V (written by TMA): boxes of 64 values x R rows, rows of 128 bytes with the 128-byte swizzle, every box on a
// 1024-byte boundary.
constexpr uint32_t kQBoxBytes = kUpCtaRows * 128;                // 64 values of all 256 rows
constexpr uint32_t kKvBoxBytes = kUpKeys * 128;                  // 64 values of 128 keys
constexpr uint32_t kKvBytes = 2 * kKvBoxBytes;                   // one K or V tile
constexpr uint32_t kOffQ = 0, kOffK = 2 * kQBoxBytes, kOffV = kOffK + 2 * kKvBytes;
constexpr uint32_t kUpSmem = kOffV + 2 * kKvBytes + 1024;        // Q | K0 K1 | V0 V1, + room to align
// tensor memory per query tile: S (128 columns; P overwrites the first 64 of them), then O (128 columns)
constexpr uint32_t kColS = 0, kColO = kUpKeys, kColsPerQTile = 256, kTmemCols = kUpQTiles * kColsPerQTile;
constexpr float kLazyLog2 = 8.0f;
constexpr uint32_t kUpWaitSpins = 1u << 18;  // tries of a wait before the CTA gives up (each suspends for a system-chosen time)

__device__ __forceinline__ float up_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Pairs of fp32 values in one 64-bit register and the arithmetic on both at once.
__device__ __forceinline__ uint64_t pack_f2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack_f2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// True in exactly one lane of a converged warp.  Unlike a comparison of the lane index, the instruction tells the compiler
// that the guarded region runs in a single thread, so descriptors and addresses of the tensor-core and copy
// instructions issued there can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t chosen;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(chosen));
  return chosen != 0;
}

// Largest power of two (at most 16) that divides the number of query heads per KV head.
__host__ __device__ inline int head_shift_of(int groups) {
  int shift = 0;
  while (shift < 4 && groups % (2 << shift) == 0) ++shift;
  return shift;
}

template <typename T>
__global__ void __launch_bounds__(kUpThreads, 1)
    gqa_prefill_umma_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q,
                            const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long bar_storage[11];  // S: tile 0, 1 | O: 0, 1 | P: 0, 1 | Q | K0 K1 | V0 V1
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;  // set by the first wait that expires; every later wait of the CTA gives up at once

  // The 256 rows of the CTA are 256 >> head_shift consecutive query positions of 1 << head_shift query heads that share
  // one KV head (row r = head r / positions, position r % positions: the order in which one TMA box of the query tensor
  // lands), so a K / V tile read from L2 serves all of them.
  const int head_shift = head_shift_of(p.groups);
  const int heads_here = 1 << head_shift;
  const int positions = kUpCtaRows >> head_shift;
  const int head_sets = p.groups >> head_shift;
  const int m0 = (int)(gridDim.x - 1 - blockIdx.x) * positions;  // tiles with the most visible keys first
  const int kvh = blockIdx.y / head_sets;
  const int hq0 = kvh * p.groups + (blockIdx.y % head_sets) * heads_here;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool softmax = threadIdx.x < kUpSoftmaxThreads;  // warps 0..7; warp 8 issues the copies and the products
  const int r_local = threadIdx.x & (kUpCtaRows - 1);  // row of the CTA; lane r_local & 127 of query tile r_local >> 7
  const int qtile = r_local >> 7;
  const int row = m0 + (r_local & (positions - 1));  // query position of this thread's row
  const int hq = hq0 + r_local / positions;

  int64_t n_keys = p.key_lengths != nullptr ? p.key_lengths[b] : p.key_len;
  n_keys = max((int64_t)0, min(n_keys, p.key_len));
  const int64_t past = n_keys - p.q_len;  // position of the chunk's first query
  const int last_row = min(m0 + positions, p.q_len) - 1;
  int64_t cta_limit = p.causal ? min(n_keys, past + last_row + 1) : n_keys;
  cta_limit = max(cta_limit, (int64_t)0);
  const int n_tiles = (int)((cta_limit + kUpKeys - 1) / kUpKeys);
  // key positions are tensor-map coordinates: they fit 32 bits
  const int n_keys32 = (int)min(n_keys, (int64_t)0x7fffffff);
  int lim = 0;  // keys this thread's row sees
  if (row < p.q_len) lim = (int)max((int64_t)0, p.causal ? min((int64_t)n_keys32, past + row + 1) : (int64_t)n_keys32);

  T* out_row = reinterpret_cast<T*>(p.out) + b * p.out_stride_b + (int64_t)hq * p.out_stride_h +
               (int64_t)row * p.out_stride_t;

  if (n_tiles == 0) {  // no row of this CTA sees a key: zeros (uniform over the CTA, nothing was allocated yet)
    if (softmax && row < p.q_len)
      for (int c = 0; c < kUpDim / 8; ++c) reinterpret_cast<uint4*>(out_row)[c] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }

  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;  // TMA boxes with the 128-byte swizzle start on 1 KB
  const uint32_t bar_s0 = smem_u32(&bar_storage[0]);  // + 8: the second query tile
  const uint32_t bar_o0 = smem_u32(&bar_storage[2]);  // + 8: the second query tile
  const uint32_t bar_p0 = smem_u32(&bar_storage[4]);  // + 8: the second query tile; one arrival per warp of the tile
  const uint32_t bar_q = smem_u32(&bar_storage[6]);
  const uint32_t bar_k0 = smem_u32(&bar_storage[7]);  // + 8: the second K stage
  const uint32_t bar_v0 = smem_u32(&bar_storage[9]);  // + 8: the second V stage
  if (threadIdx.x == 0) {
    for (int i = 0; i < 11; ++i) mbar_init(bar_s0 + 8 * i, (i == 4 || i == 5) ? kUpRows / 32 : 1);
    abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, kTmemCols);

  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  // Bounded wait that also ends as soon as another thread of the CTA has given up.  Called by whole warps; the answer
  // is the same in every lane, so the warp-wide tensor-memory instructions behind it never run in a part of a warp.
  auto wait = [&](uint32_t bar, int use) -> bool {  // `use`: how many times the barrier completed before this phase
    const uint32_t parity = (uint32_t)(use & 1);
    bool landed = false;
    for (uint32_t spin = 0; spin < kUpWaitSpins && !landed; ++spin) {
      uint32_t done;
      asm volatile(  // no suspend-time hint: with one the waits of a healthy CTA were measured 4 % slower
          "{\n"
          ".reg .pred p;\n"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
          "selp.u32 %0, 1, 0, p;\n"
          "}\n"
          : "=r"(done)
          : "r"(bar), "r"(parity)
          : "memory");
      landed = done != 0;
      if (!landed && *(volatile int*)&abort_flag != 0) break;
    }
    if (!landed) *(volatile int*)&abort_flag = 1;
    return __all_sync(0xffffffffu, landed);
  };

  if (!softmax) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kUpIssuerRegs));
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kUpSoftmaxRegs));
  }
  if (!softmax) {
    if (warp == kUpSoftmaxThreads / 32) {
    // ---- issuing warp: the whole warp walks the loop, one elected lane issues -----------------------------------------
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? kUmmaBF16 : kUmmaF16;
    constexpr uint32_t idesc_s = umma_idesc(kFmt, kFmt, false, false, kUpRows, kUpKeys);
    constexpr uint32_t idesc_o = umma_idesc(kFmt, kFmt, false, true, kUpRows, kUpDim);
    // Descriptors of the first 16-wide K step of every operand; a later step, stage or query tile is the same
    // descriptor with its byte offset (in 16-byte units) added to the address field.  Q and K: K-major rows of 128
    // bytes (eight rows = 1024 bytes); V: MN-major, the next 64 values of head_dim are the next box.
    const uint64_t desc_q = umma_smem_desc_sw128(smem + kOffQ, 16, 1024);
    const uint64_t desc_k = umma_smem_desc_sw128(smem + kOffK, 16, 1024);
    const uint64_t desc_v = umma_smem_desc_sw128(smem + kOffV, kKvBoxBytes, 1024);
    // The stage of a tile (tile & 1), the query tile and "first tile" are compile-time constants in everything below (the
    // loop over the tiles is unrolled by two): descriptors, tensor-memory addresses and barrier addresses are then
    // loop-invariant bases plus constants, which the compiler keeps in uniform registers.  With the stage taken from the
    // loop counter every product cost about 125 clocks to issue, twice the 64 it takes the tensor pipe to execute.
    // Two boxes (the two halves of head_dim) per tile, counted in bytes on the stage's barrier; a tile past the last
    // one is not loaded and never waited for.
    auto load_k = [&](auto stage_c, int tile) {
      constexpr int kStage = decltype(stage_c)::value;
      if (tile >= n_tiles || !elect_one()) return;
      const uint32_t bar = bar_k0 + kStage * 8, dst = smem + kOffK + kStage * kKvBytes;
      mbar_expect_tx(bar, kKvBytes);
      tma_load_4d(dst, &map_k, 0, tile * kUpKeys, kvh, b, bar);
      tma_load_4d(dst + kKvBoxBytes, &map_k, 64, tile * kUpKeys, kvh, b, bar);
    };
    auto load_v = [&](auto stage_c, int tile) {
      constexpr int kStage = decltype(stage_c)::value;
      if (tile >= n_tiles || !elect_one()) return;
      const uint32_t bar = bar_v0 + kStage * 8, dst = smem + kOffV + kStage * kKvBytes;
      mbar_expect_tx(bar, kKvBytes);
      tma_load_4d(dst, &map_v, 0, tile * kUpKeys, kvh, b, bar);
      tma_load_4d(dst + kKvBoxBytes, &map_v, 64, tile * kUpKeys, kvh, b, bar);
    };
    // S_qt = Q_qt . K(stage)^T into the score columns of query tile qt
    auto issue_scores = [&](auto qt_c, auto stage_c) {
      constexpr int kQt = decltype(qt_c)::value, kStage = decltype(stage_c)::value;
      if (!elect_one()) return;
      tcgen05_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kUpDim / 16; ++k)  // 16 values of K per instruction: 32 bytes of a row, four steps per box
        umma_f16(tmem + kQt * kColsPerQTile + kColS,
                 desc_q + (uint64_t)(((k / 4) * kQBoxBytes + kQt * (kUpRows * 128) + (k % 4) * 32) >> 4),
                 desc_k + (uint64_t)((kStage * kKvBytes + (k / 4) * kKvBoxBytes + (k % 4) * 32) >> 4), idesc_s,
                 k > 0 ? 1u : 0u);
      umma_commit(bar_s0 + kQt * 8);
    };
    // O_qt += P_qt . V(stage): P sits in the first 64 score columns (two keys per column)
    auto issue_values = [&](auto qt_c, auto stage_c, auto first_c) {
      constexpr int kQt = decltype(qt_c)::value, kStage = decltype(stage_c)::value;
      constexpr bool kFirst = decltype(first_c)::value;
      if (!elect_one()) return;
      tcgen05_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kUpKeys / 16; ++k)  // 16 keys per instruction: eight columns of P, 16 rows of V = 2048 bytes
        umma_f16_ts(tmem + kQt * kColsPerQTile + kColO, tmem + kQt * kColsPerQTile + kColS + 8 * k,
                    desc_v + (uint64_t)((kStage * kKvBytes + k * 16 * 128) >> 4), idesc_o, (!kFirst || k > 0) ? 1u : 0u);
      umma_commit(bar_o0 + kQt * 8);
    };
    using Zero = std::integral_constant<int, 0>;
    using One = std::integral_constant<int, 1>;
    if (elect_one()) {
      mbar_expect_tx(bar_q, 2 * kQBoxBytes);  // positions past the chunk's end arrive as zeros
      tma_load_4d(smem + kOffQ, &map_q, 0, m0, hq0, b, bar_q);
      tma_load_4d(smem + kOffQ + kQBoxBytes, &map_q, 64, m0, hq0, b, bar_q);
    }
    load_k(Zero{}, 0);
    load_v(Zero{}, 0);
    load_k(One{}, 1);
    load_v(One{}, 1);
    bool ok = wait(bar_q, 0) && wait(bar_k0, 0);
    if (ok) {
      issue_scores(Zero{}, Zero{});
      issue_scores(One{}, Zero{});
    }
    // Order on the tensor pipe: ... P0.V | S0(next) | P1.V | S1(next) ...  The pipe runs in issue order, so S_qt(next)
    // overwrites the columns of P_qt only after the product that reads them, and while the threads of one query tile
    // are busy with their softmax the pipe works for the other tile.
    auto step = [&](auto stage_c, auto first_c, int it) -> bool {
      constexpr int kStage = decltype(stage_c)::value;  // it & 1
      using Next = std::integral_constant<int, 1 - kStage>;
      // query tile 0: P_0(it) is in tensor memory and O_0 rescaled; V(it) has landed
      if (!wait(bar_p0, it) || !wait(bar_v0 + kStage * 8, it >> 1)) return false;
      issue_values(Zero{}, stage_c, first_c);
      if (it + 1 < n_tiles) {
        if (!wait(bar_k0 + (1 - kStage) * 8, (it + 1) >> 1)) return false;
        issue_scores(Zero{}, Next{});
      }
      // query tile 1
      if (!wait(bar_p0 + 8, it)) return false;
      issue_values(One{}, stage_c, first_c);
      if (it + 1 < n_tiles) issue_scores(One{}, Next{});
      // both softmaxes have read their S(it): the K stage is free; the V stage once the second product is complete
      load_k(stage_c, it + 2);
      if (it + 2 < n_tiles) {
        if (!wait(bar_o0 + 8, it)) return false;
        load_v(stage_c, it + 2);
      }
      return true;
    };
    if (ok) ok = step(Zero{}, std::true_type{}, 0);
    int it = 1;
    for (; ok && it + 1 < n_tiles; it += 2) {
      ok = step(One{}, std::false_type{}, it);
      if (ok) ok = step(Zero{}, std::false_type{}, it + 1);
    }
    if (ok && it < n_tiles) ok = step(One{}, std::false_type{}, it);
    }
  } else {
    // ---- softmax warps: thread t owns row t; warps 0..3 query tile 0, warps 4..7 query tile 1 --------------------------
    const uint32_t t_lane = tmem_addr(tmem, 32 * (warp & 3), qtile * kColsPerQTile);
    const uint32_t t_s = t_lane + kColS;
    const uint32_t t_o = t_lane + kColO;
    const uint32_t my_s = bar_s0 + qtile * 8, my_o = bar_o0 + qtile * 8, my_p = bar_p0 + qtile * 8;
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int key0 = it * kUpKeys;  // first key of the tile
      const int visible = max(0, min(kUpKeys, lim - key0));  // keys of the tile this row sees
      constexpr int kChunk = 32;  // score columns per tensor-memory load
      ok = wait(my_s, it);
      if (!ok) break;
      tcgen05_fence_after_sync();

      // The whole row of S into registers (four loads in flight, one wait), mask, row maximum
      uint32_t x[kUpKeys];
#pragma unroll
      for (int c = 0; c < kUpKeys / kChunk; ++c) tmem_ld32(t_s + kChunk * c, *reinterpret_cast<uint32_t(*)[kChunk]>(&x[kChunk * c]));
      tmem_wait_ld();
      if (visible < kUpKeys) {
#pragma unroll
        for (int i = 0; i < kUpKeys; ++i)
          if (i >= visible) x[i] = 0xff800000u;  // -inf: exp2 gives 0
      }
      float mx4[4] = {__uint_as_float(x[0]), __uint_as_float(x[1]), __uint_as_float(x[2]), __uint_as_float(x[3])};
#pragma unroll
      for (int i = 4; i + 8 <= kUpKeys; i += 8) {  // two new values per instruction
        mx4[0] = max3(mx4[0], __uint_as_float(x[i]), __uint_as_float(x[i + 1]));
        mx4[1] = max3(mx4[1], __uint_as_float(x[i + 2]), __uint_as_float(x[i + 3]));
        mx4[2] = max3(mx4[2], __uint_as_float(x[i + 4]), __uint_as_float(x[i + 5]));
        mx4[3] = max3(mx4[3], __uint_as_float(x[i + 6]), __uint_as_float(x[i + 7]));
      }
      mx4[0] = max3(mx4[0], __uint_as_float(x[kUpKeys - 4]), __uint_as_float(x[kUpKeys - 3]));
      mx4[1] = max3(mx4[1], __uint_as_float(x[kUpKeys - 2]), __uint_as_float(x[kUpKeys - 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;  // the scale is positive

      // Lazy running maximum (log2 units): it moves only when it would grow by more than 2^8, and only then is the row
      // of O rescaled, for which the previous product has to be complete
      const bool grew = mx > m_run + kLazyLog2;
      if (__any_sync(0xffffffffu, grew)) {  // tcgen05.ld / st are warp-wide
        const float alpha = grew ? up_ex2(m_run - mx) : 1.0f;  // 0 while m_run is -inf
        if (grew) m_run = mx;
        l_run *= alpha;
        if (it > 0) {
          ok = wait(my_o, it - 1);
          if (!ok) break;
          tcgen05_fence_after_sync();
#pragma unroll 1
          for (int cc = 0; cc < kUpDim / 16; ++cc) {
            uint32_t o[16];
            tmem_ld16(t_o + 16 * cc, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st16(t_o + 16 * cc, o);
          }
        }
      }
      const float m_ref = m_run == -INFINITY ? 0.0f : m_run;

      // P = exp2(S * scale - m) as 16-bit pairs over the scores (keys 32c .. 32c + 31 into columns 16c .. 16c + 15),
      // row sum; the scaling and the sums run on pairs of values (one instruction for two)
      const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2), shift2 = pack_f2(-m_ref, -m_ref);
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};  // four pairs of +0.0f
#pragma unroll
      for (int c = 0; c < kUpKeys / kChunk; ++c) {
        uint32_t packed[kChunk / 2];
#pragma unroll
        for (int j = 0; j < kChunk / 2; ++j) {
          const int i = kChunk * c + 2 * j;
          const uint64_t arg = fma2(pack_f2(__uint_as_float(x[i]), __uint_as_float(x[i + 1])), scale2, shift2);
          float lo, hi;
          unpack_f2(arg, lo, hi);
          lo = up_ex2(lo);  // exp2(-inf) = 0 for hidden keys
          hi = up_ex2(hi);
          sum2[j % 4] = add2(sum2[j % 4], pack_f2(lo, hi));
          packed[j] = pack2<T>(lo, hi);
        }
        tmem_st16(t_s + (kChunk / 2) * c, packed);
      }
      float sum4[4];
      {
        const uint64_t total = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
        unpack_f2(total, sum4[0], sum4[1]);
        sum4[2] = sum4[3] = 0.0f;
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_wait_st();

      // In the tile that holds the last key the V rows behind it may hold anything (they are inside the tensor but past
      // this row's length), and 0 x NaN would poison O, so the threads of query tile 0 (whose product is issued first)
      // zero them (whole 128-byte rows: the swizzle permutes inside a row)
      if (qtile == 0 && key0 + kUpKeys > n_keys32) {
        ok = wait(bar_v0 + (it & 1) * 8, it >> 1);
        if (!ok) break;
        const int first = max(0, n_keys32 - key0);
        uint8_t* v_stage = smem_raw + (smem - smem_u32(smem_raw)) + kOffV + (it & 1) * kKvBytes;
        for (int i = threadIdx.x; i < (kUpKeys - first) * 16; i += kUpRows) {
          const int r = first + (i >> 4), piece = i & 15;  // 8 pieces of 16 bytes in each of the two boxes
          *reinterpret_cast<uint4*>(v_stage + (piece >> 3) * kKvBoxBytes + r * 128 + (piece & 7) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        fence_async_smem();
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p);
    }
    if (ok) ok = wait(my_o, n_tiles - 1);
    if (ok) {
      tcgen05_fence_after_sync();
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
      for (int c = 0; c < kUpDim / 16; ++c) {
        uint32_t r[16];
        tmem_ld16(t_o + 16 * c, r);
        tmem_wait_ld();
        if (row < p.q_len) {
          uint4 lo, hi;
          lo.x = pack2<T>(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
          lo.y = pack2<T>(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
          lo.z = pack2<T>(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
          lo.w = pack2<T>(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
          hi.x = pack2<T>(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
          hi.y = pack2<T>(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
          hi.z = pack2<T>(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
          hi.w = pack2<T>(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
          reinterpret_cast<uint4*>(out_row)[2 * c] = lo;
          reinterpret_cast<uint4*>(out_row)[2 * c + 1] = hi;
        }
      }
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag != 0) atomicAdd(&g_prefill_umma_faults, 1);
  if (warp == 0) tmem_free(tmem, kTmemCols);
}

// ---- head_dim 256 ------------------------------------------------------------------------------------------------------
// O alone fills half of tensor memory (256 columns), so a CTA owns ONE 128-row query tile and the other half holds two
// score buffers of 64 columns: S(t + 1) is computed while the threads work on tile t, and the only thing the tensor
// pipe ever waits for is P.  64-key tiles (a K or V tile is 32 KB; two stages of each and Q make 192 KB).  Warp 4 issues
// the products, warp 5 the copies (eight boxes and two byte counts per tile: on the issuing warp they would cost more
// than the products of the tile), warps 0..3 are the softmax, thread t = row t.
// With two query tiles per CTA (256 rows per K / V tile, 256 columns of tensor memory per query tile, eight softmax
// warps) the same structure serves head_dim 64 (`WideCfg<64, 2>`).  `WideCfg<128, 2>` is correct too, but takes 1.10 ms
// on the case the kernel above takes 1.03 ms for, so it is not instantiated.
template <int D, int QT>
struct WideCfg {
  static constexpr int kDim = D, kRows = 128, kCtaRows = QT * 128, kKeys = 64, kStages = 2;
  static constexpr int kSoftmaxWarps = 4 * QT;
  static constexpr int kThreads = (kSoftmaxWarps + 2 + 3) / 4 * 4 * 32;  // softmax warps, issuing warp, copy warp
  static constexpr uint32_t kKvBoxBytes = kKeys * 128;              // 64 values of 64 keys
  static constexpr uint32_t kKvBytes = (D / 64) * kKvBoxBytes;      // one K or V tile
  static constexpr uint32_t kOffK = 0, kOffV = kOffK + kStages * kKvBytes;
  static constexpr uint32_t kSmem = kOffV + kStages * kKvBytes + 1024;
  // tensor memory per query tile: S0 | S1 (64 columns each) | O (D columns) | Q (D / 2 columns, two values each).  Q is
  // the A operand of S = Q . K^T and is read from tensor memory: a 128 x 64 x 16 product that fetches its 4 KB A operand
  // from shared memory took about 76 clocks here instead of 32, and those products bounded the kernel.
  static constexpr uint32_t kColS = 0, kColO = 2 * kKeys, kColQ = kColO + D, kColsPerQTile = D <= 128 ? 256 : 512;
  static constexpr uint32_t kTmemCols = 512;
  static_assert(kColQ + D / 2 <= kColsPerQTile && QT * kColsPerQTile <= 512, "tensor memory layout");
};

template <typename T, int D, int QT>
__global__ void __launch_bounds__((WideCfg<D, QT>::kThreads), 1)
    gqa_prefill_umma_wide_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q,
                               const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  using Cfg = WideCfg<D, QT>;
  constexpr int kWdDim = Cfg::kDim, kWdRows = Cfg::kRows, kWdKeys = Cfg::kKeys;
  constexpr uint32_t kWdKvBoxBytes = Cfg::kKvBoxBytes, kWdKvBytes = Cfg::kKvBytes;
  constexpr uint32_t kWdOffK = Cfg::kOffK, kWdOffV = Cfg::kOffV, kWdColS = Cfg::kColS, kWdColO = Cfg::kColO, kWdColQ = Cfg::kColQ;
  constexpr uint32_t kWdTmemCols = Cfg::kTmemCols, kColsQ = Cfg::kColsPerQTile;
  constexpr int kSoftmaxWarps = Cfg::kSoftmaxWarps;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long bar_storage[6 * QT + 5];  // S, P, O [query tile][tile parity] | Q | K landed [stage] | V landed [stage]
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int head_shift = head_shift_of(p.groups);
  const int heads_here = 1 << head_shift;
  const int positions = Cfg::kCtaRows >> head_shift;
  const int head_sets = p.groups >> head_shift;
  const int m0 = (int)(gridDim.x - 1 - blockIdx.x) * positions;  // tiles with the most visible keys first
  const int kvh = blockIdx.y / head_sets;
  const int hq0 = kvh * p.groups + (blockIdx.y % head_sets) * heads_here;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r_local = threadIdx.x & (Cfg::kCtaRows - 1);
  const int qtile = r_local >> 7;
  const int row = m0 + (r_local & (positions - 1));  // query position of this thread's row
  const int hq = hq0 + r_local / positions;

  int64_t n_keys = p.key_lengths != nullptr ? p.key_lengths[b] : p.key_len;
  n_keys = max((int64_t)0, min(n_keys, p.key_len));
  const int64_t past = n_keys - p.q_len;
  const int last_row = min(m0 + positions, p.q_len) - 1;
  int64_t cta_limit = p.causal ? min(n_keys, past + last_row + 1) : n_keys;
  cta_limit = max(cta_limit, (int64_t)0);
  const int n_tiles = (int)((cta_limit + kWdKeys - 1) / kWdKeys);
  const int n_keys32 = (int)min(n_keys, (int64_t)0x7fffffff);
  int lim = 0;  // keys this thread's row sees
  if (row < p.q_len) lim = (int)max((int64_t)0, p.causal ? min((int64_t)n_keys32, past + row + 1) : (int64_t)n_keys32);
  T* out_row = reinterpret_cast<T*>(p.out) + b * p.out_stride_b + (int64_t)hq * p.out_stride_h +
               (int64_t)row * p.out_stride_t;

  if (n_tiles == 0) {  // no row of this CTA sees a key: zeros (uniform over the CTA, nothing was allocated yet)
    if (warp < kSoftmaxWarps && row < p.q_len)
      for (int c = 0; c < kWdDim / 8; ++c) reinterpret_cast<uint4*>(out_row)[c] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }

  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_s0 = smem_u32(&bar_storage[0]);  // + 16 * query tile + 8 * (tile & 1) for S, P and O
  const uint32_t bar_p0 = smem_u32(&bar_storage[2 * QT]);
  const uint32_t bar_o0 = smem_u32(&bar_storage[4 * QT]);
  const uint32_t bar_q = smem_u32(&bar_storage[6 * QT]);
  const uint32_t bar_k0 = smem_u32(&bar_storage[6 * QT + 1]);  // + 8 * stage
  const uint32_t bar_v0 = smem_u32(&bar_storage[6 * QT + 3]);
  if (threadIdx.x == 0) {
    for (int i = 0; i < 6 * QT + 5; ++i)
      mbar_init(bar_s0 + 8 * i, (i >= 2 * QT && i < 4 * QT) ? kWdRows / 32 : (i == 6 * QT ? kSoftmaxWarps : 1));
    abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, kWdTmemCols);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  auto wait = [&](uint32_t bar, int use) -> bool {  // as in the head_dim 128 kernel
    const uint32_t parity = (uint32_t)(use & 1);
    bool landed = false;
    for (uint32_t spin = 0; spin < kUpWaitSpins && !landed; ++spin) {
      uint32_t done;
      asm volatile(
          "{\n"
          ".reg .pred p;\n"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
          "selp.u32 %0, 1, 0, p;\n"
          "}\n"
          : "=r"(done)
          : "r"(bar), "r"(parity)
          : "memory");
      landed = done != 0;
      if (!landed && *(volatile int*)&abort_flag != 0) break;
    }
    if (!landed) *(volatile int*)&abort_flag = 1;
    return __all_sync(0xffffffffu, landed);
  };
  using Zero = std::integral_constant<int, 0>;
  using One = std::integral_constant<int, 1>;

  if (warp == kSoftmaxWarps + 1) {
    // ---- copies: K(t) goes where K(t - 2) was once S(t - 2) is complete, V(t) where V(t - 2) was once P.V(t - 2) is --
    // (the waits come in the order the tensor pipe completes them: S(t - 2), P.V(t - 2), S(t - 1), ...)
    auto load_tile = [&](auto stage_c, int t, bool keys) {
      constexpr int kStage = decltype(stage_c)::value;
      if (!elect_one()) return;
      const uint32_t bar = (keys ? bar_k0 : bar_v0) + kStage * 8;
      const uint32_t dst = smem + (keys ? kWdOffK : kWdOffV) + kStage * kWdKvBytes;
      mbar_expect_tx(bar, kWdKvBytes);
#pragma unroll
      for (int i = 0; i < kWdDim / 64; ++i)
        tma_load_4d(dst + i * kWdKvBoxBytes, keys ? &map_k : &map_v, 64 * i, t * kWdKeys, kvh, b, bar);
    };
    bool ok = true;
    auto produce = [&](auto stage_c, int t) {
      constexpr int kStage = decltype(stage_c)::value;  // t & 1
      if (t >= 2) ok = wait(bar_s0 + (QT - 1) * 16 + kStage * 8, (t - 2) >> 1);
      if (!ok) return;
      load_tile(stage_c, t, true);
      if (t >= 2) ok = wait(bar_o0 + (QT - 1) * 16 + kStage * 8, (t - 2) >> 1);
      if (!ok) return;
      load_tile(stage_c, t, false);
    };
    for (int t = 0; t < n_tiles && ok; t += 2) {
      produce(Zero{}, t);
      if (ok && t + 1 < n_tiles) produce(One{}, t + 1);
    }
  } else if (warp == kSoftmaxWarps) {
    // ---- products -----------------------------------------------------------------------------------------------------
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? kUmmaBF16 : kUmmaF16;
    constexpr uint32_t idesc_s = umma_idesc(kFmt, kFmt, false, false, kWdRows, kWdKeys);
    constexpr uint32_t idesc_o = umma_idesc(kFmt, kFmt, false, true, kWdRows, kWdDim);
    const uint64_t desc_k = umma_smem_desc_sw128(smem + kWdOffK, 16, 1024);
    const uint64_t desc_v = umma_smem_desc_sw128(smem + kWdOffV, kWdKvBoxBytes, 1024);  // next 64 values: next box
    auto issue_scores = [&](auto qt_c, auto stage_c) {
      constexpr int kQt = decltype(qt_c)::value, kStage = decltype(stage_c)::value;  // stage = score buffer
      if (!elect_one()) return;
      tcgen05_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kWdDim / 16; ++k)  // 16 values of K per instruction: 32 bytes of a row, four steps per box
        umma_f16_ts(tmem + kQt * kColsQ + kWdColS + kStage * kWdKeys, tmem + kQt * kColsQ + kWdColQ + 8 * k,
                    desc_k + (uint64_t)((kStage * kWdKvBytes + (k / 4) * kWdKvBoxBytes + (k % 4) * 32) >> 4), idesc_s,
                    k > 0 ? 1u : 0u);
      umma_commit(bar_s0 + kQt * 16 + kStage * 8);
    };
    auto issue_values = [&](auto qt_c, auto stage_c, auto first_c) {
      constexpr int kQt = decltype(qt_c)::value, kStage = decltype(stage_c)::value;
      constexpr bool kFirst = decltype(first_c)::value;
      if (!elect_one()) return;
      tcgen05_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kWdKeys / 16; ++k)  // 16 keys per instruction: eight columns of P, 16 rows of V = 2048 bytes
        umma_f16_ts(tmem + kQt * kColsQ + kWdColO, tmem + kQt * kColsQ + kWdColS + kStage * kWdKeys + 8 * k,
                    desc_v + (uint64_t)((kStage * kWdKvBytes + k * 16 * 128) >> 4), idesc_o, (!kFirst || k > 0) ? 1u : 0u);
      umma_commit(bar_o0 + kQt * 16 + kStage * 8);
    };
    bool ok = wait(bar_q, 0) && wait(bar_k0, 0);
    if (ok) {
      issue_scores(Zero{}, Zero{});
      if constexpr (QT == 2) issue_scores(One{}, Zero{});
    }
    auto step = [&](auto stage_c, auto first_c, int t) -> bool {
      constexpr int kStage = decltype(stage_c)::value;
      using Next = std::integral_constant<int, 1 - kStage>;
      if (t + 1 < n_tiles) {  // S(t + 1): its buffer held P(t - 1), which the product issued before this one has read
        if (!wait(bar_k0 + (1 - kStage) * 8, (t + 1) >> 1)) return false;
        issue_scores(Zero{}, Next{});
        if constexpr (QT == 2) issue_scores(One{}, Next{});
      }
      if (!wait(bar_p0 + kStage * 8, t >> 1) || !wait(bar_v0 + kStage * 8, t >> 1)) return false;
      issue_values(Zero{}, stage_c, first_c);
      if constexpr (QT == 2) {
        if (!wait(bar_p0 + 16 + kStage * 8, t >> 1)) return false;
        issue_values(One{}, stage_c, first_c);
      }
      return true;
    };
    if (ok) ok = step(Zero{}, std::true_type{}, 0);
    int t = 1;
    for (; ok && t + 1 < n_tiles; t += 2) {
      ok = step(One{}, std::false_type{}, t);
      if (ok) ok = step(Zero{}, std::false_type{}, t + 1);
    }
    if (ok && t < n_tiles) ok = step(One{}, std::false_type{}, t);
  } else if (warp < kSoftmaxWarps) {
    // ---- softmax: thread t owns row t -----------------------------------------------------------------------------------
    constexpr int kChunk = 32;
    const uint32_t t_lane = tmem_addr(tmem, 32 * (warp & 3), qtile * kColsQ);
    const uint32_t my_s0 = bar_s0 + qtile * 16, my_p0 = bar_p0 + qtile * 16, my_o0 = bar_o0 + qtile * 16;
    const uint32_t t_o = t_lane + kWdColO;
    {
      // this thread's row of Q into tensor memory (two values per column, as the A operand of the score products
      // expects them); rows past the chunk's end are zeros
      const uint4* q_row = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) + b * p.q_stride_b +
                                                         (int64_t)hq * p.q_stride_h + (int64_t)row * p.q_stride_t);
#pragma unroll 2
      for (int c = 0; c < kWdDim / 32; ++c) {  // 32 values = 64 bytes = 16 columns
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 v = row < p.q_len ? q_row[4 * c + j] : make_uint4(0u, 0u, 0u, 0u);
          w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
        tmem_st16(t_lane + kWdColQ + 16 * c, w);
      }
      tmem_wait_st();
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_q);
    }
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      const int key0 = it * kWdKeys;
      const int visible = max(0, min(kWdKeys, lim - key0));
      const uint32_t t_s = t_lane + kWdColS + (it & 1) * kWdKeys;
      ok = wait(my_s0 + (it & 1) * 8, it >> 1);
      if (!ok) break;
      tcgen05_fence_after_sync();
      uint32_t x[kWdKeys];
#pragma unroll
      for (int c = 0; c < kWdKeys / kChunk; ++c) tmem_ld32(t_s + kChunk * c, *reinterpret_cast<uint32_t(*)[kChunk]>(&x[kChunk * c]));
      tmem_wait_ld();
      if (visible < kWdKeys) {
#pragma unroll
        for (int i = 0; i < kWdKeys; ++i)
          if (i >= visible) x[i] = 0xff800000u;  // -inf: exp2 gives 0
      }
      float mx4[4] = {__uint_as_float(x[0]), __uint_as_float(x[1]), __uint_as_float(x[2]), __uint_as_float(x[3])};
#pragma unroll
      for (int i = 4; i + 8 <= kWdKeys; i += 8) {
        mx4[0] = max3(mx4[0], __uint_as_float(x[i]), __uint_as_float(x[i + 1]));
        mx4[1] = max3(mx4[1], __uint_as_float(x[i + 2]), __uint_as_float(x[i + 3]));
        mx4[2] = max3(mx4[2], __uint_as_float(x[i + 4]), __uint_as_float(x[i + 5]));
        mx4[3] = max3(mx4[3], __uint_as_float(x[i + 6]), __uint_as_float(x[i + 7]));
      }
      mx4[0] = max3(mx4[0], __uint_as_float(x[kWdKeys - 4]), __uint_as_float(x[kWdKeys - 3]));
      mx4[1] = max3(mx4[1], __uint_as_float(x[kWdKeys - 2]), __uint_as_float(x[kWdKeys - 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;  // the scale is positive
      const bool grew = mx > m_run + kLazyLog2;
      if (__any_sync(0xffffffffu, grew)) {  // tcgen05.ld / st are warp-wide
        const float alpha = grew ? up_ex2(m_run - mx) : 1.0f;  // 0 while m_run is -inf
        if (grew) m_run = mx;
        l_run *= alpha;
        if (it > 0) {  // the row of O, for which the previous product has to be complete
          ok = wait(my_o0 + ((it - 1) & 1) * 8, (it - 1) >> 1);
          if (!ok) break;
          tcgen05_fence_after_sync();
#pragma unroll 1
          for (int cc = 0; cc < kWdDim / 16; ++cc) {
            uint32_t o[16];
            tmem_ld16(t_o + 16 * cc, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st16(t_o + 16 * cc, o);
          }
        }
      }
      const float m_ref = m_run == -INFINITY ? 0.0f : m_run;
      const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2), shift2 = pack_f2(-m_ref, -m_ref);
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < kWdKeys / kChunk; ++c) {
        uint32_t packed[kChunk / 2];
#pragma unroll
        for (int j = 0; j < kChunk / 2; ++j) {
          const int i = kChunk * c + 2 * j;
          const uint64_t arg = fma2(pack_f2(__uint_as_float(x[i]), __uint_as_float(x[i + 1])), scale2, shift2);
          float lo, hi;
          unpack_f2(arg, lo, hi);
          lo = up_ex2(lo);
          hi = up_ex2(hi);
          sum2[j % 4] = add2(sum2[j % 4], pack_f2(lo, hi));
          packed[j] = pack2<T>(lo, hi);
        }
        tmem_st16(t_s + (kChunk / 2) * c, packed);
      }
      float s_lo, s_hi;
      unpack_f2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), s_lo, s_hi);
      l_run += s_lo + s_hi;
      tmem_wait_st();
      // the V rows behind the last key may hold anything: zero them in the tile that straddles it (see the other kernel)
      if (qtile == 0 && key0 + kWdKeys > n_keys32) {
        ok = wait(bar_v0 + (it & 1) * 8, it >> 1);
        if (!ok) break;
        const int first = max(0, n_keys32 - key0);
        uint8_t* v_stage = smem_raw + (smem - smem_u32(smem_raw)) + kWdOffV + (it & 1) * kWdKvBytes;
        constexpr int kPieces = kWdDim / 8;  // 16-byte pieces per key: 8 in each box
        for (int i = threadIdx.x; i < (kWdKeys - first) * kPieces; i += kWdRows) {
          const int r = first + i / kPieces, piece = i % kPieces;
          *reinterpret_cast<uint4*>(v_stage + (piece >> 3) * kWdKvBoxBytes + r * 128 + (piece & 7) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        fence_async_smem();
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p0 + (it & 1) * 8);
    }
    if (ok) ok = wait(my_o0 + ((n_tiles - 1) & 1) * 8, (n_tiles - 1) >> 1);
    if (ok) {
      tcgen05_fence_after_sync();
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll 4
      for (int c = 0; c < kWdDim / 16; ++c) {
        uint32_t r[16];
        tmem_ld16(t_o + 16 * c, r);
        tmem_wait_ld();
        if (row < p.q_len) {
          uint4 lo, hi;
          lo.x = pack2<T>(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
          lo.y = pack2<T>(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
          lo.z = pack2<T>(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
          lo.w = pack2<T>(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
          hi.x = pack2<T>(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
          hi.y = pack2<T>(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
          hi.z = pack2<T>(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
          hi.w = pack2<T>(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
          reinterpret_cast<uint4*>(out_row)[2 * c] = lo;
          reinterpret_cast<uint4*>(out_row)[2 * c + 1] = hi;
        }
      }
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag != 0) atomicAdd(&g_prefill_umma_faults, 1);
  if (warp == 0) tmem_free(tmem, kWdTmemCols);
}

}  // namespace

bool prefill_umma_applicable(const PrefillParams& p, int head_dim, int dtype) {
  static const bool disabled = [] {
    const char* flag = std::getenv("ANNA_B200_PREFILL_UMMA");
    return flag != nullptr && flag[0] == '0';
  }();
  if (disabled) return false;
  if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || (dtype != ANNA_DTYPE_F16 && dtype != ANNA_DTYPE_BF16))
    return false;
  // the output rows are written as 16-byte vectors
  if (p.out_stride_b % 8 != 0 || p.out_stride_h % 8 != 0 || p.out_stride_t % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(p.out) & 15u) != 0) return false;
  if (p.key_len <= 0) return false;
  // The rows of a CTA are query positions x the heads that share a KV head (a power of two, at most 16): chunks that
  // fill less than half a CTA's rows (and are shorter than 64 positions) leave most of the tile empty, and the mma.sync
  // kernel serves them.
  const int cta_rows = head_dim == 256 ? 128 : 256;
  return p.q_len >= 64 || (int64_t)p.q_len * (1 << head_shift_of(p.groups)) * 2 >= cta_rows;
}

// Tensor map of a [B, H, L, dim] 16-bit tensor given by element strides, seen as (dim, L, H, B).
static bool prefill_tensor_map(CUtensorMap* out, const void* base, int64_t len, int heads, int batch, int64_t stride_t,
                               int64_t stride_h, int64_t stride_b, uint32_t box_len, uint32_t box_heads,
                               int dim = kUpDim) {
  if (len <= 0 || heads <= 0 || batch <= 0) return false;
  const uint64_t extents[4] = {(uint64_t)dim, (uint64_t)len, (uint64_t)heads, (uint64_t)batch};
  uint64_t strides[3] = {(uint64_t)stride_t * 2, (uint64_t)stride_h * 2, (uint64_t)stride_b * 2};
  const uint64_t used[3] = {(uint64_t)len, (uint64_t)heads, (uint64_t)batch};
  for (int i = 0; i < 3; ++i) {
    if (used[i] == 1 && strides[i] == 0) strides[i] = 256;  // never stepped along
    if (strides[i] == 0 || strides[i] % 16 != 0 || strides[i] >= ((uint64_t)1 << 40)) return false;
  }
  const uint32_t box[4] = {64, box_len, box_heads, 1};
  return encode_map_16bit(out, base, 4, extents, strides, box);
}

template <typename T>
static int launch_prefill_umma_t(const PrefillParams& p, int batch, int q_heads, cudaStream_t stream) {
  auto kernel = gqa_prefill_umma_kernel<T>;
  const int head_shift = head_shift_of(p.groups);
  const int positions = kUpCtaRows >> head_shift;
  CUtensorMap map_q, map_k, map_v;
  const int kv_heads = q_heads / p.groups;
  if (!prefill_tensor_map(&map_q, p.q, p.q_len, q_heads, batch, p.q_stride_t, p.q_stride_h, p.q_stride_b,
                          (uint32_t)positions, 1u << head_shift) ||
      !prefill_tensor_map(&map_k, p.k, p.key_len, kv_heads, batch, p.kv_stride_t, p.kv_stride_h, p.kv_stride_b, kUpKeys, 1) ||
      !prefill_tensor_map(&map_v, p.v, p.key_len, kv_heads, batch, p.kv_stride_t, p.kv_stride_h, p.kv_stride_b, kUpKeys, 1))
    return kPrefillNotServed;  // no encoder in this driver, or a layout it refuses: the mma.sync kernel takes over
  static bool configured[64] = {};
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !configured[device]) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kUpSmem));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  dim3 grid((unsigned)((p.q_len + positions - 1) / positions), (unsigned)(q_heads >> head_shift), (unsigned)batch);
  kernel<<<grid, kUpThreads, kUpSmem, stream>>>(p, map_q, map_k, map_v);
  return check_launch("gqa_prefill_umma_kernel");
}

template <typename T, int D, int QT>
static int launch_prefill_umma_wide_t(const PrefillParams& p, int batch, int q_heads, cudaStream_t stream) {
  using Cfg = WideCfg<D, QT>;
  auto kernel = gqa_prefill_umma_wide_kernel<T, D, QT>;
  const int head_shift = head_shift_of(p.groups);
  const int positions = Cfg::kCtaRows >> head_shift;
  CUtensorMap map_q, map_k, map_v;
  const int kv_heads = q_heads / p.groups;
  if (!prefill_tensor_map(&map_q, p.q, p.q_len, q_heads, batch, p.q_stride_t, p.q_stride_h, p.q_stride_b,
                          (uint32_t)positions, 1u << head_shift, D) ||
      !prefill_tensor_map(&map_k, p.k, p.key_len, kv_heads, batch, p.kv_stride_t, p.kv_stride_h, p.kv_stride_b, Cfg::kKeys, 1,
                          D) ||
      !prefill_tensor_map(&map_v, p.v, p.key_len, kv_heads, batch, p.kv_stride_t, p.kv_stride_h, p.kv_stride_b, Cfg::kKeys, 1,
                          D))
    return kPrefillNotServed;
  static bool configured[64] = {};
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !configured[device]) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::kSmem));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  dim3 grid((unsigned)((p.q_len + positions - 1) / positions), (unsigned)(q_heads >> head_shift), (unsigned)batch);
  kernel<<<grid, Cfg::kThreads, Cfg::kSmem, stream>>>(p, map_q, map_k, map_v);
  return check_launch("gqa_prefill_umma_wide_kernel");
}

int launch_prefill_umma(const PrefillParams& p, int batch, int q_heads, int head_dim, int dtype, cudaStream_t stream) {
  if (head_dim == 256)
    return dtype == ANNA_DTYPE_BF16 ? launch_prefill_umma_wide_t<__nv_bfloat16, 256, 1>(p, batch, q_heads, stream)
                                    : launch_prefill_umma_wide_t<__half, 256, 1>(p, batch, q_heads, stream);
  if (head_dim == 64)
    return dtype == ANNA_DTYPE_BF16 ? launch_prefill_umma_wide_t<__nv_bfloat16, 64, 2>(p, batch, q_heads, stream)
                                    : launch_prefill_umma_wide_t<__half, 64, 2>(p, batch, q_heads, stream);
  return dtype == ANNA_DTYPE_BF16 ? launch_prefill_umma_t<__nv_bfloat16>(p, batch, q_heads, stream)
                                  : launch_prefill_umma_t<__half>(p, batch, q_heads, stream);
}

int prefill_umma_faults(int* count) {
  int32_t value = 0;
  ANNA_CUDA_CHECK(cudaMemcpyFromSymbol(&value, g_prefill_umma_faults, sizeof(value)));
  *count = (int)value;
  return ANNA_OK;
}

}  // namespace anna
