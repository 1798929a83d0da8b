// Split pass of single-token GQA decode over packed TurboQuant pages on the 5th-generation tensor cores
// (tcgen05.mma, accumulators and the de-quantized key operand in tensor memory).  head_dim 128, 3- or 4-bit codes,
// 16-token pages, value groups of 32, up to 4 query heads per kv head; other shapes take the mma.sync kernel.
//
// A CTA (8 warps) owns one (row, kv head, chunk of the packed prefix) and walks it in steps of 128 tokens:
//
//   packed pages --bulk copy (cp.async.bulk, mbarrier)--> shared, 2 stages of 8 page tiles
//   keys:   thread = (token, half of the coordinates).  Code nibbles / 2-bit fields select bytes of an e4m3 centroid
//           table with one byte-permute per four codes (rounded centroid and rounding residual); sign bits sit in
//           the selector bit that makes the permute replicate the top bit of the chosen byte, which turns a table of
//           1.0 bytes into {1.0, 0.0}.  The bytes go straight to tensor memory (tcgen05.st): token = lane, 128 bytes
//           per plane, so the score products read their A operand from tensor memory and nothing de-quantized ever
//           crosses shared memory.
//   S1[128 tok x 16] = centroid(K) . Q1^T (+ residual terms)     S2 = sign(K) . Q2^T     (tcgen05.mma kind::f8f6f4)
//   scores: thread = (token, two heads) reads its S1 / S2 cells back (tcgen05.ld), forms norm * (S1 + rnorm * S2),
//           p = 2^(score - m) against a per-head reference maximum shared by the CTA (raised, with a rescale of the
//           accumulators, only when a score exceeds it by 2^8), and writes B[token][head, group] = p * value scale
//           as f16 into shared memory; sum p and sum p * zero point stay in registers.
//   values: 4-bit codes are masked in place into f16 bit patterns (a nibble in the low mantissa bits is the
//           subnormal code * 2^-24 or * 2^-20), one logic op per two values, and stored token-major in shared memory
//   O^T[128 dims x 16 (head, group)] += V^T . B                              (tcgen05.mma kind::f16, MN-major operands)
//           every dim row only uses the 4 columns of its own value group; the power of two of its nibble position
//           and the zero-point sums are applied when the partial is written.
//
// Every wait on the copy engine or the tensor core is bounded (mbarrier_utils.cuh); when one expires the CTA counts a
// fault, skips the rest of its chunk, still frees its tensor memory and leaves.
#include "fused_combine.cuh"
#include "tq_common.cuh"
#include "tq_decode_params.cuh"
#include "umma_utils.cuh"

#include <cuda_fp8.h>

#include <cstdlib>
#include <type_traits>

namespace anna {

__device__ int32_t g_tq_umma_faults;  // bumped when a bounded wait of the kernel below expires

constexpr int kUmmaThreads = 256;
constexpr int kUmmaWarps = kUmmaThreads / 32;
constexpr int kUmmaStepTokens = 128;
constexpr int kUmmaTiles = kUmmaStepTokens / 16;
constexpr int kUmmaDim = 128;
constexpr int kUmmaHeads = 4;            // query heads per kv head served by one CTA
constexpr int kUmmaStages = 3;           // input stages (steps of 128 tokens in flight or being read)
constexpr float kUmmaFp8Top = 224.0f;    // largest magnitude of a scaled query entry (e4m3 holds up to 448)
constexpr float kUmmaLazy = 8.0f;        // log2 units the reference maximum may lag behind
constexpr int kUmmaQueryConsts = 32;     // floats behind the query operand: 1/qs [0..3], S2 start values [16..19]

template <typename T, int BITS>
struct UmmaCfg {
  static_assert(BITS == 3 || BITS == 4, "tensor-memory TurboQuant decode is built for 3- and 4-bit codes");
  static constexpr int D = kUmmaDim;
  static constexpr int kGroups = D / 32;
  static constexpr int kKeyBytes = D * BITS / 8;
  static constexpr int kIdxBytes = BITS == 3 ? D / 4 : kKeyBytes;
  static constexpr int kValBytes = D / 2;
  // layout of one 16-token page chunk (= tq_make_layout for 16-token pages): codes, norms, residual norms, value
  // codes, scales, zeros
  static constexpr int kOffKey = 0;
  static constexpr int kOffNorm = 16 * kKeyBytes;
  static constexpr int kOffRnorm = kOffNorm + 64;
  static constexpr int kOffVal = kOffRnorm + 64;
  static constexpr int kOffScale = kOffVal + 16 * kValBytes;
  static constexpr int kOffZero = kOffScale + 16 * kGroups * 2;
  static constexpr int kTileDataBytes = kOffZero + 16 * kGroups * 2;
  static constexpr int kTileStride = (kTileDataBytes + 127) / 128 * 128;
  // shared memory map
  static constexpr int kStageBytes = kUmmaTiles * kTileStride;
  static constexpr int kOffStages = 0;
  static constexpr uint32_t kVSbo = 144, kVLbo = 16 * kVSbo;       // V^T, MN-major: 16 dim groups per 8 tokens
  static constexpr int kOffV = kOffStages + kUmmaStages * kStageBytes;
  static constexpr int kVBytes = 16 * kVLbo;
  static constexpr uint32_t kBSbo = 128, kBLbo = 256;              // B = p * scale, MN-major: 2 column groups per 8 tokens
  static constexpr int kOffB = kOffV + kVBytes;
  static constexpr int kBBytes = 16 * kBLbo;
  static constexpr uint32_t kQSbo = 128, kQLbo = 256;              // query planes, K-major: 16 rows per 16 K bytes
  static constexpr int kQPlane = 8 * kQLbo;
  static constexpr int kOffQ = kOffB + kBBytes;
  static constexpr int kQBytes = 3 * kQPlane + kUmmaQueryConsts * 4;
  static constexpr int kOffMisc = kOffQ + kQBytes;
  static constexpr int kMiscBytes = 1024;
  static constexpr int kSmemBytes = kOffMisc + kMiscBytes;
  // tensor memory columns (32-bit cells): three key planes of 128 bytes per token, two score accumulators, O
  static constexpr uint32_t kColKey = 0, kColS1 = 96, kColS2 = 112, kColO = 128, kColumns = 256;
};

// Coordinate that sits in byte `slot` (0..127) of a token's row of the index plane / the sign plane, i.e. the order
// in which the kernel's byte permutes emit the codes of a token.
template <int BITS>
__device__ __forceinline__ int umma_idx_slot_coord(int slot) {
  if constexpr (BITS == 4) return slot;  // nibbles come out in order
  // 2-bit fields, 16 per word: even fields of the low / high half-word, then the odd ones
  const int word = slot / 16, kind = (slot % 16) / 4, j = slot % 4;
  return 16 * word + ((kind & 1) ? 8 : 0) + 2 * j + (kind >> 1);
}
template <int BITS>
__device__ __forceinline__ int umma_sign_slot_coord(int slot) {
  if constexpr (BITS == 4) return slot;
  // 1-bit plane, 32 per word: register pair k (0..3) takes bits 3 - k + 4j of the low and of the high half-word
  const int word = slot / 32, k = (slot % 32) / 8, half = (slot % 8) / 4, j = slot % 4;
  return 32 * word + 16 * half + 4 * j + 3 - k;
}

__device__ __forceinline__ uint32_t umma_f32_to_e4m3(float x) {
  return (uint32_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float umma_e4m3_to_f32(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(__half(h));
}
// Byte permute in PTX's default mode: result byte i is the byte of {a (0-3), b (4-7)} that bits 0-2 of nibble i of
// `sel` name, or, when bit 3 of that nibble is set, eight copies of that byte's top bit.
__device__ __forceinline__ uint32_t umma_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// Four bytes {1.0, 0.0} (e4m3) for bit 3 of the low four nibbles of `sel` being {0, 1}.
__device__ __forceinline__ uint32_t umma_one_minus_bit3(uint32_t sel) {
  return umma_prmt(0x38383838u, 0x38383838u, sel);
}
// 32 bytes (8 words) from shared memory as two 16-byte loads.
__device__ __forceinline__ void lds_pair16(const uint8_t* ptr, uint32_t (&w)[8]) {
  const uint4 a = reinterpret_cast<const uint4*>(ptr)[0];
  const uint4 b = reinterpret_cast<const uint4*>(ptr)[1];
  w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
  w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}
__device__ __forceinline__ float umma_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void umma_wait_prior_grids() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem], e4m3 operands: A is 128 lanes x 8 columns (32 bytes of K per row).
__device__ __forceinline__ void umma_f8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------------------------------------------------------------
// Rotates the (up to 4) queries of one (row, kv head) and writes the B operand of the score products as the kernel
// wants it in shared memory: three K-major planes of 16 rows x 128 e4m3 bytes (Q1 rounded, Q1 rounding residual, Q2
// rounded; rows beyond the group are zero; byte order = the order in which the kernel emits a token's codes), then
// per head 1 / qs and the start value of S2.
//   score (log2 units) = norm * (S1 + rnorm * S2) / qs,   Q1 = fwht(s1*q) * f1 * qs,   Q2 = -2 * fwht(s2*fwht(s1*q)) * f2 * qs
// The sign plane holds 1.0 for a clear bit: sum_d q_d * (2 bit_d - 1) = sum_d q_d - 2 sum_d q_d a_d, so Q2 carries the
// factor -2 and S2 starts at -1/2 of the sum of the rounded Q2 bytes.  qs brings the largest entry to 224.
template <typename T, int BITS>
__global__ void __launch_bounds__(128) tq_prepare_queries_umma_kernel(const TqDecodeParams p) {
  using Cfg = UmmaCfg<T, BITS>;
  constexpr int D = kUmmaDim, E = D / 32;
  __shared__ __align__(16) uint8_t image[Cfg::kQBytes];
  __shared__ uint8_t vals[kUmmaHeads][3][kUmmaDim];  // [head][Q1 rounded, Q1 residual, Q2 rounded][coordinate]
  const int kvh = blockIdx.x;
  const int b = blockIdx.y;
  const int g_count = min(kUmmaHeads, p.groups);
  const int hq0 = kvh * p.groups;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < Cfg::kQBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(image)[i] = 0u;
  __syncthreads();
  float* consts = reinterpret_cast<float*>(image + 3 * Cfg::kQPlane);
  if (threadIdx.x < kUmmaHeads) consts[threadIdx.x] = 1.0f;  // heads beyond the group: any positive factor
  const T* q_ptr = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b;
  const float inv_sqrt_d = rsqrt_dim_const<D>();
  const float log2e = 1.4426950408889634f;
  const float f1 = p.scaling * log2e * inv_sqrt_d * inv_sqrt_d;
  const float f2 = -2.0f * p.scaling * log2e * 1.2533141373155001f * inv_sqrt_d * inv_sqrt_d * inv_sqrt_d;
  if (warp < g_count) {
    const int g = warp;
    float w[E], w2[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int d = lane * E + j;
      w[j] = ElemTraits<T>::to_float(q_ptr[(int64_t)(hq0 + g) * p.q_stride_h + d]);
      if (p.signs1[d] < 0.0f) w[j] = -w[j];
    }
    warp_fwht<E>(w, lane);
#pragma unroll
    for (int j = 0; j < E; ++j) {
      w2[j] = w[j];
      if (p.signs2[lane * E + j] < 0.0f) w2[j] = -w2[j];
    }
    warp_fwht<E>(w2, lane);
    float top = 0.0f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      w[j] *= f1;
      w2[j] *= f2;
      top = fmaxf(top, fmaxf(fabsf(w[j]), fabsf(w2[j])));
    }
#pragma unroll
    for (int dl = 1; dl < 32; dl <<= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, dl));
    const float qs = (top > 1e-30f && top < 1e30f) ? kUmmaFp8Top / top : 1.0f;
    // the bytes go through shared memory by coordinate first: byte `slot` of a plane holds coordinate slot_coord(slot)
    float sum2 = 0.0f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int d = lane * E + j;
      const float v1 = w[j] * qs, v2 = w2[j] * qs;
      const uint32_t h1 = umma_f32_to_e4m3(v1), h2 = umma_f32_to_e4m3(v2);
      const uint32_t l1 = umma_f32_to_e4m3(v1 - umma_e4m3_to_f32(h1));
      vals[g][0][d] = (uint8_t)h1;
      vals[g][1][d] = (uint8_t)l1;
      vals[g][2][d] = (uint8_t)h2;
      sum2 += umma_e4m3_to_f32(h2);
    }
#pragma unroll
    for (int dl = 1; dl < 32; dl <<= 1) sum2 += __shfl_xor_sync(0xffffffffu, sum2, dl);
    __syncwarp();
    for (int slot = lane; slot < D; slot += 32) {
      const int ci = umma_idx_slot_coord<BITS>(slot), cs = umma_sign_slot_coord<BITS>(slot);
      const int off = (slot / 16) * (int)Cfg::kQLbo + (g / 8) * (int)Cfg::kQSbo + (g % 8) * 16 + slot % 16;
      image[0 * Cfg::kQPlane + off] = vals[g][0][ci];
      image[1 * Cfg::kQPlane + off] = vals[g][1][ci];
      image[2 * Cfg::kQPlane + off] = vals[g][2][cs];
    }
    if (lane == 0) {
      consts[g] = 1.0f / qs;
      consts[16 + g] = -0.5f * sum2;
    }
  }
  __syncthreads();
  uint32_t* out = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(p.query_frags) +
                                              ((int64_t)b * gridDim.x + kvh) * Cfg::kQBytes);
  for (int i = threadIdx.x; i < Cfg::kQBytes / 4; i += blockDim.x) out[i] = reinterpret_cast<const uint32_t*>(image)[i];
}

// ---------------------------------------------------------------------------------------------------------------------
template <typename T, int BITS>
__global__ void __launch_bounds__(kUmmaThreads, 2) tq_decode_umma_kernel(const TqDecodeParams p) {
  using Cfg = UmmaCfg<T, BITS>;
  constexpr int D = kUmmaDim;
  extern __shared__ __align__(1024) uint8_t smem_raw[];

  const int slot = blockIdx.x;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int g_count = min(kUmmaHeads, p.groups);
  const int hq0 = kvh * p.groups;

  int64_t len64 = p.lengths[b];
  len64 = max((int64_t)0, min(len64, p.max_len));
  const int len = (int)len64;
  const int R = p.residual_len;
  const int Lq = len > R ? len - R : 0;
  const int win = len - Lq;
  const int active_window = (win + p.chunk_tokens - 1) / p.chunk_tokens;
  const int active_packed = (Lq + p.chunk_tokens - 1) / p.chunk_tokens;
  const int active_chunks = active_window + active_packed;
  const int chunk = slot - p.num_window_chunks;
  const int t0 = chunk * p.chunk_tokens;
  if (len == 0 || chunk < 0 || t0 >= Lq) {  // window chunks run in tq_window_split_mma_kernel
    umma_wait_prior_grids();
    return;
  }
  const int t1 = min(Lq, t0 + p.chunk_tokens);
  const int out_slot = active_window + chunk;  // active slots stay contiguous: [window | packed]
  const int num_tiles = (t1 - t0 + 15) / 16;
  const int num_steps = (num_tiles + kUmmaTiles - 1) / kUmmaTiles;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int quad = warp & 3;                 // tensor-memory lane quadrant of this warp
  const int half = warp >> 2;                // which half of the coordinates / heads this thread handles
  const int tok = quad * 32 + lane;          // token of the step (= tensor-memory lane) this thread serves

  uint8_t* s_stage = smem_raw + Cfg::kOffStages;
  uint8_t* s_v = smem_raw + Cfg::kOffV;
  uint8_t* s_b = smem_raw + Cfg::kOffB;
  uint8_t* s_q = smem_raw + Cfg::kOffQ;
  uint8_t* s_misc = smem_raw + Cfg::kOffMisc;
  // misc: [0,32) full barriers of the stages, [32,40) scores done, [40,48) values done, [48,56) query operand,
  // [56,60) tensor-memory address, [64,192) valid tokens per tile and stage, [192,320) block maxima, [320,..) sums
  const uint32_t bar_full = smem_u32(s_misc);
  const uint32_t bar_s = smem_u32(s_misc + 32);
  const uint32_t bar_o = smem_u32(s_misc + 40);
  const uint32_t bar_q = smem_u32(s_misc + 48);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_misc + 56);
  volatile int* stage_valid = reinterpret_cast<volatile int*>(s_misc + 64);   // [stages][8]
  float* s_max = reinterpret_cast<float*>(s_misc + 192);                       // [8 warps][2], then 4 old references
  float* s_sum = reinterpret_cast<float*>(s_misc + 320);                       // [8 warps][10]

  if (threadIdx.x == 0) {
    for (int i = 0; i < kUmmaStages; ++i) mbar_init(bar_full + i * 8, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_init(bar_q, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(tmem_slot, Cfg::kColumns);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  const int32_t* table_row = p.block_table + (int64_t)b * p.table_stride;
  // Start the copies of one step (8 consecutive page tiles) into a stage: lanes 0..7 of warp 0 look up and copy one
  // tile each, lane 0 arms the stage's barrier with the bytes of all of them first.
  auto issue_step = [&](int step, int stage) {
    int valid = 0;
    const uint8_t* chunk_ptr = nullptr;
    if (lane < kUmmaTiles) {
      const int tile = step * kUmmaTiles + lane;
      if (tile < num_tiles) {
        const int ts = t0 + tile * 16;
        const int32_t pid = table_row[ts >> 4];
        if (pid >= 0 && pid < p.num_pages) {  // else a hole in the block table: nothing to copy
          valid = min(16, t1 - ts);
          chunk_ptr = p.pages + ((int64_t)pid * p.kv_heads + kvh) * p.layout.chunk_bytes;
        }
      }
      stage_valid[stage * kUmmaTiles + lane] = valid;
    }
    const uint32_t bar = bar_full + stage * 8;
    const unsigned have = __ballot_sync(0xffffffffu, valid > 0);
    if (lane == 0) {
      if (have != 0u) mbar_expect_tx(bar, (uint32_t)__popc(have) * Cfg::kTileDataBytes);
      else mbar_arrive(bar);
    }
    __syncwarp();
    if (valid > 0)
      bulk_copy_g2s(smem_u32(s_stage + stage * Cfg::kStageBytes + lane * Cfg::kTileStride), chunk_ptr,
                    Cfg::kTileDataBytes, bar);
  };
  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_q, Cfg::kQBytes);
      bulk_copy_g2s(smem_u32(s_q),
                    static_cast<const uint8_t*>(p.query_frags) + ((int64_t)b * gridDim.y + kvh) * Cfg::kQBytes,
                    Cfg::kQBytes, bar_q);
    }
    __syncwarp();
    for (int i = 0; i < kUmmaStages && i < num_steps; ++i) issue_step(i, i);
  }

  // centroid byte tables for the byte permutes: e4m3 rounding of each centroid and of what the rounding left over
  uint32_t lut_hi[2] = {0u, 0u}, lut_lo[2] = {0u, 0u};
  {
    constexpr int kEntries = 1 << (BITS - 1);
#pragma unroll
    for (int e = 0; e < kEntries; ++e) {
      const float c = __ldg(p.centroids + e);
      const uint32_t hi = umma_f32_to_e4m3(c);
      const uint32_t lo = umma_f32_to_e4m3(c - umma_e4m3_to_f32(hi));
      lut_hi[e / 4] |= hi << (8 * (e % 4));
      lut_lo[e / 4] |= lo << (8 * (e % 4));
    }
    if constexpr (BITS == 3) {
      lut_hi[1] = lut_hi[0];
      lut_lo[1] = lut_lo[0];
    }
  }

  bool failed = !mbar_wait(bar_q, 0u);
  const float* qconst = reinterpret_cast<const float*>(s_q + 3 * Cfg::kQPlane);
  // this thread's two score columns are heads 2 * half and 2 * half + 1
  const float kq[2] = {qconst[2 * half], qconst[2 * half + 1]};
  const float s2_init[2] = {qconst[16 + 2 * half], qconst[16 + 2 * half + 1]};

  // running state: reference maxima (fragment units: true log2 score = kq * x), sum of p, sum of p * zero point
  float m_ref[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  float z_run[2][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int g = 0; g < 4; ++g) z_run[h][g] = 0.0f;

  constexpr uint32_t kIdescScore = umma_idesc(kUmmaE4M3, kUmmaE4M3, false, false, 128, 16);
  constexpr uint32_t kIdescValue = umma_idesc(kUmmaF16, kUmmaF16, true, true, 128, 16);
  const uint32_t q_addr = smem_u32(s_q);
  const uint32_t v_addr = smem_u32(s_v);
  const uint32_t b_addr = smem_u32(s_b);
  const uint32_t my_lanes = (uint32_t)(quad * 32);

  // byte offsets of this thread's token inside a stage, and of its outputs (all loop-invariant)
  const int tok_tile = (tok >> 4) * Cfg::kTileStride, tok_row = tok & 15;
  const int off_keys = tok_tile + Cfg::kOffKey + tok_row * Cfg::kKeyBytes;
  const int off_norm = tok_tile + Cfg::kOffNorm + tok_row * 4;
  const int off_rnorm = tok_tile + Cfg::kOffRnorm + tok_row * 4;
  const int off_scale = tok_tile + Cfg::kOffScale + tok_row * 8;
  const int off_zero = tok_tile + Cfg::kOffZero + tok_row * 8;
  uint8_t* const b_dst = s_b + (tok >> 3) * Cfg::kBLbo + half * Cfg::kBSbo + (tok & 7) * 16;
  // values: warp w owns tile w of a step; lanes 0-15 / 16-31 take the 16 dim groups of two tokens per round
  const int off_vsrc = warp * Cfg::kTileStride + Cfg::kOffVal + (lane >> 4) * Cfg::kValBytes + (lane & 15) * 4;
  uint8_t* const v_dst = s_v + (2 * warp) * Cfg::kVLbo + (lane & 15) * Cfg::kVSbo + (lane >> 4) * 16;

  // Per-token metadata of a step (norm, residual norm, value scales and zero points of this thread's token).
  struct TokenMeta {
    float norm, rnorm, vs[4], vz[4];
    bool valid;
  };
  auto load_meta = [&](int stage, TokenMeta& m) {
    const uint8_t* st = s_stage + stage * Cfg::kStageBytes;
    m.valid = tok_row < stage_valid[stage * kUmmaTiles + (tok >> 4)];
    m.norm = m.rnorm = 0.0f;
#pragma unroll
    for (int g = 0; g < 4; ++g) m.vs[g] = m.vz[g] = 0.0f;
    if (!m.valid) return;
    m.norm = *reinterpret_cast<const float*>(st + off_norm);
    m.rnorm = *reinterpret_cast<const float*>(st + off_rnorm);
    const uint2 sw = *reinterpret_cast<const uint2*>(st + off_scale);
    const uint2 zw = *reinterpret_cast<const uint2*>(st + off_zero);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      m.vs[0] = __uint_as_float(sw.x << 16); m.vs[1] = __uint_as_float(sw.x & 0xffff0000u);
      m.vs[2] = __uint_as_float(sw.y << 16); m.vs[3] = __uint_as_float(sw.y & 0xffff0000u);
      m.vz[0] = __uint_as_float(zw.x << 16); m.vz[1] = __uint_as_float(zw.x & 0xffff0000u);
      m.vz[2] = __uint_as_float(zw.y << 16); m.vz[3] = __uint_as_float(zw.y & 0xffff0000u);
    } else {
      const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sw.x));
      const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sw.y));
      const float2 z01 = __half22float2(*reinterpret_cast<const __half2*>(&zw.x));
      const float2 z23 = __half22float2(*reinterpret_cast<const __half2*>(&zw.y));
      m.vs[0] = s01.x; m.vs[1] = s01.y; m.vs[2] = s23.x; m.vs[3] = s23.y;
      m.vz[0] = z01.x; m.vz[1] = z01.y; m.vz[2] = z23.x; m.vz[3] = z23.y;
    }
  };
  // Keys of this thread's token: its 64 coordinates (k-steps 2 * half, 2 * half + 1) -> e4m3 bytes in tensor memory.
  auto dequant_keys = [&](int stage) {
    const uint8_t* krow = s_stage + stage * Cfg::kStageBytes + off_keys;
    if constexpr (BITS == 4) {
      uint32_t w[8];
      lds_pair16(krow + half * 32, w);
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        // one plane after the other: the eight registers of a store are produced back to back
        const uint32_t col = Cfg::kColKey + (uint32_t)(2 * half + ks) * 8;
        uint32_t t[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) t[i] = w[4 * ks + i] & 0x77777777u;
        {
          uint32_t r[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            r[2 * i] = umma_prmt(lut_hi[0], lut_hi[1], t[i]);
            r[2 * i + 1] = umma_prmt(lut_hi[0], lut_hi[1], t[i] >> 16);
          }
          tmem_st8(tmem_addr(tmem, my_lanes, col), r);
        }
        {
          uint32_t r[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            r[2 * i] = umma_prmt(lut_lo[0], lut_lo[1], t[i]);
            r[2 * i + 1] = umma_prmt(lut_lo[0], lut_lo[1], t[i] >> 16);
          }
          tmem_st8(tmem_addr(tmem, my_lanes, col + 32), r);
        }
        {
          uint32_t r[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            r[2 * i] = umma_one_minus_bit3(w[4 * ks + i]);
            r[2 * i + 1] = umma_one_minus_bit3(w[4 * ks + i] >> 16);
          }
          tmem_st8(tmem_addr(tmem, my_lanes, col + 64), r);
        }
      }
    } else {
      uint32_t w[4], sw2[2];
      {
        const uint4 v = *reinterpret_cast<const uint4*>(krow + half * 16);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        const uint2 sgn = *reinterpret_cast<const uint2*>(krow + Cfg::kIdxBytes + half * 8);
        sw2[0] = sgn.x; sw2[1] = sgn.y;
      }
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        uint32_t hi[8], lo[8], sg[8];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t x = w[2 * ks + i];
          const uint32_t e = x & 0x33333333u, o = (x >> 2) & 0x33333333u;
          hi[4 * i + 0] = umma_prmt(lut_hi[0], lut_hi[1], e);
          hi[4 * i + 1] = umma_prmt(lut_hi[0], lut_hi[1], e >> 16);
          hi[4 * i + 2] = umma_prmt(lut_hi[0], lut_hi[1], o);
          hi[4 * i + 3] = umma_prmt(lut_hi[0], lut_hi[1], o >> 16);
          lo[4 * i + 0] = umma_prmt(lut_lo[0], lut_lo[1], e);
          lo[4 * i + 1] = umma_prmt(lut_lo[0], lut_lo[1], e >> 16);
          lo[4 * i + 2] = umma_prmt(lut_lo[0], lut_lo[1], o);
          lo[4 * i + 3] = umma_prmt(lut_lo[0], lut_lo[1], o >> 16);
        }
        const uint32_t x = sw2[ks];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          sg[2 * k] = umma_one_minus_bit3(x << k);
          sg[2 * k + 1] = umma_one_minus_bit3(x >> (16 - k));
        }
        const uint32_t col = Cfg::kColKey + (uint32_t)(2 * half + ks) * 8;
        tmem_st8(tmem_addr(tmem, my_lanes, col), hi);
        tmem_st8(tmem_addr(tmem, my_lanes, col + 32), lo);
        tmem_st8(tmem_addr(tmem, my_lanes, col + 64), sg);
      }
    }
    tmem_wait_st();
  };
  // Score products of the step whose keys sit in tensor memory; issued by one thread.
  auto issue_scores = [&]() {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint32_t a_hi = tmem + Cfg::kColKey + ks * 8, a_lo = a_hi + 32, a_sg = a_hi + 64;
      const uint32_t qoff = q_addr + 2 * ks * Cfg::kQLbo;
      const uint64_t q1h = umma_smem_desc(qoff, Cfg::kQLbo, Cfg::kQSbo);
      const uint64_t q1l = umma_smem_desc(qoff + Cfg::kQPlane, Cfg::kQLbo, Cfg::kQSbo);
      const uint64_t q2h = umma_smem_desc(qoff + 2 * Cfg::kQPlane, Cfg::kQLbo, Cfg::kQSbo);
      umma_f8_ts(tmem + Cfg::kColS1, a_hi, q1h, kIdescScore, ks > 0);
      umma_f8_ts(tmem + Cfg::kColS1, a_hi, q1l, kIdescScore, 1u);
      umma_f8_ts(tmem + Cfg::kColS1, a_lo, q1h, kIdescScore, 1u);
      umma_f8_ts(tmem + Cfg::kColS2, a_sg, q2h, kIdescScore, ks > 0);
    }
    umma_commit(bar_s);
  };

  // ---- software pipeline: while the tensor core scores step n + 1, the threads finish step n (softmax, values) ---------
  TokenMeta cur;
  if (!mbar_wait(bar_full, 0u)) failed = true;
  load_meta(0, cur);
  dequant_keys(0);
  tcgen05_fence_before_sync();
  {
    const int any_failed = __syncthreads_or(failed ? 1 : 0);
    tcgen05_fence_after_sync();
    if (any_failed) failed = true;
  }
  if (threadIdx.x == 0 && !failed) issue_scores();

  for (int n = 0; n < num_steps && !failed; ++n) {
    const int stage = n % kUmmaStages;
    // ---- scores of step n out of tensor memory ------------------------------------------------------------------------
    if (!mbar_wait(bar_s, (uint32_t)n & 1u)) failed = true;
    tcgen05_fence_after_sync();
    float sc[2] = {-INFINITY, -INFINITY};
    {
      uint32_t r1[4], r2[4];
      tmem_ld4(tmem_addr(tmem, my_lanes, Cfg::kColS1), r1);
      tmem_ld4(tmem_addr(tmem, my_lanes, Cfg::kColS2), r2);
      tmem_wait_ld();
      if (cur.valid) {
        const float a0 = __uint_as_float(half ? r1[2] : r1[0]), a1 = __uint_as_float(half ? r1[3] : r1[1]);
        const float c0 = __uint_as_float(half ? r2[2] : r2[0]), c1 = __uint_as_float(half ? r2[3] : r2[1]);
        sc[0] = cur.norm * fmaf(cur.rnorm, c0 + s2_init[0], a0);
        sc[1] = cur.norm * fmaf(cur.rnorm, c1 + s2_init[1], a1);
      }
    }
    // ---- keys of step n + 1 into tensor memory (the score products of step n are done with it) ---------------------------
    TokenMeta next;
    next.valid = false;
    const bool more = n + 1 < num_steps;
    if (more) {
      const int next_stage = (n + 1) % kUmmaStages;
      if (!failed && !mbar_wait(bar_full + next_stage * 8, (uint32_t)((n + 1) / kUmmaStages) & 1u)) failed = true;
      load_meta(next_stage, next);
      dequant_keys(next_stage);
    }
    // the reference maxima move only when some score exceeds them by more than 2^8 (true units)
    const bool grew = ((sc[0] - m_ref[0]) * kq[0] > kUmmaLazy) || ((sc[1] - m_ref[1]) * kq[1] > kUmmaLazy);
    tcgen05_fence_before_sync();
    const int votes = __syncthreads_or((grew ? 1 : 0) | (failed ? 2 : 0));
    tcgen05_fence_after_sync();
    if (votes & 2) { failed = true; break; }
    if (threadIdx.x == 0 && more) issue_scores();

    if (votes & 1) {
      // block maximum per head -> new reference; everything accumulated so far shrinks by 2^(kq * (old - new))
      float mx[2] = {sc[0], sc[1]};
#pragma unroll
      for (int dl = 1; dl < 32; dl <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], dl));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], dl));
      }
      if (lane == 0) {
        s_max[warp * 2] = mx[0];
        s_max[warp * 2 + 1] = mx[1];
        if (quad == 0) {  // old references of this thread's two heads
          s_max[16 + 2 * half] = m_ref[0];
          s_max[16 + 2 * half + 1] = m_ref[1];
        }
      }
      // the value products of step n - 1 must be complete before O is rescaled
      if (n > 0 && !mbar_wait(bar_o, (uint32_t)(n - 1) & 1u)) failed = true;
      tcgen05_fence_after_sync();
      __syncthreads();
      float f_own[2];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int h = 2 * half + h2;
        float neu = s_max[16 + h];
#pragma unroll
        for (int w = 0; w < 4; ++w) neu = fmaxf(neu, s_max[(half * 4 + w) * 2 + h2]);
        f_own[h2] = (neu == -INFINITY) ? 1.0f : umma_exp2(kq[h2] * (m_ref[h2] - neu));  // old = -inf gives 0
        m_ref[h2] = neu;
        l_run[h2] *= f_own[h2];
#pragma unroll
        for (int g = 0; g < 4; ++g) z_run[h2][g] *= f_own[h2];
      }
      if (n > 0) {
        // O in tensor memory: this thread rescales columns [8 * half, +8) of its lane = heads 2 * half, 2 * half + 1
        uint32_t o[8];
        tmem_ld8(tmem_addr(tmem, my_lanes, Cfg::kColO + 8 * half), o);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 8; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f_own[c >> 2]);
        tmem_st8(tmem_addr(tmem, my_lanes, Cfg::kColO + 8 * half), o);
        tmem_wait_st();
      }
      __syncthreads();  // s_max may be reused by the next rescale
    }

    // ---- p, B = p * value scale, running sums; value codes of step n -> shared memory -------------------------------------
    // (B and the value operand are free again once the value products of step n - 1 are done)
    if (n > 0 && !failed && !mbar_wait(bar_o, (uint32_t)(n - 1) & 1u)) failed = true;
    tcgen05_fence_after_sync();
    {
      float pr[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float nm = m_ref[h] == -INFINITY ? 0.0f : -kq[h] * m_ref[h];
        pr[h] = cur.valid ? umma_exp2(fmaf(sc[h], kq[h], nm)) : 0.0f;
        l_run[h] += pr[h];
#pragma unroll
        for (int g = 0; g < 4; ++g) z_run[h][g] = fmaf(pr[h], cur.vz[g], z_run[h][g]);
      }
      // columns n = head * 4 + group; this thread's heads are 2 * half, 2 * half + 1 -> column group `half`
      uint4 out;
      out.x = pack2<__half>(pr[0] * cur.vs[0], pr[0] * cur.vs[1]);
      out.y = pack2<__half>(pr[0] * cur.vs[2], pr[0] * cur.vs[3]);
      out.z = pack2<__half>(pr[1] * cur.vs[0], pr[1] * cur.vs[1]);
      out.w = pack2<__half>(pr[1] * cur.vs[2], pr[1] * cur.vs[3]);
      *reinterpret_cast<uint4*>(b_dst) = out;
    }
    {
      const uint8_t* vsrc = s_stage + stage * Cfg::kStageBytes + off_vsrc;
#pragma unroll
      for (int i = 0; i < 8; ++i) {  // round i: tokens 2i and 2i + 1 of the tile
        const uint32_t x = *reinterpret_cast<const uint32_t*>(vsrc + i * 2 * Cfg::kValBytes);
        const uint32_t y = x >> 8;
        // f16 bit patterns: a nibble in mantissa bits 0-3 is code * 2^-24, in bits 4-7 code * 2^-20
        const uint4 out = make_uint4(x & 0x000F000Fu, x & 0x00F000F0u, y & 0x000F000Fu, y & 0x00F000F0u);
        *reinterpret_cast<uint4*>(v_dst + (i >> 2) * Cfg::kVLbo + (i & 3) * 32) = out;
      }
    }
    fence_async_smem();
    tcgen05_fence_before_sync();
    __syncthreads();  // B and the values are in shared memory; the stage of step n has been read completely
    tcgen05_fence_after_sync();
    if (warp == 0) {
      const bool warp_failed = __any_sync(0xffffffffu, failed);
      if (lane == 0 && !warp_failed) {
#pragma unroll
        for (int k = 0; k < kUmmaStepTokens / 16; ++k)
          umma_f16(tmem + Cfg::kColO, umma_smem_desc(v_addr + 2 * k * Cfg::kVLbo, Cfg::kVLbo, Cfg::kVSbo),
                   umma_smem_desc(b_addr + 2 * k * Cfg::kBLbo, Cfg::kBLbo, Cfg::kBSbo), kIdescValue,
                   (n > 0 || k > 0) ? 1u : 0u);
        umma_commit(bar_o);
      }
      __syncwarp();
      if (n + kUmmaStages < num_steps && !warp_failed) issue_step(n + kUmmaStages, stage);  // this stage is free again
    }
    cur = next;
  }


  // ---- all products done; gather the sums ---------------------------------------------------------------------------
  const int steps_done = failed ? 0 : num_steps;
  if (steps_done > 0 && !mbar_wait(bar_o, (uint32_t)(steps_done - 1) & 1u)) failed = true;
  tcgen05_fence_after_sync();
  if (failed && threadIdx.x == 0) atomicAdd(&g_tq_umma_faults, 1);
  {
    float vals[10] = {l_run[0], l_run[1], z_run[0][0], z_run[0][1], z_run[0][2], z_run[0][3],
                      z_run[1][0], z_run[1][1], z_run[1][2], z_run[1][3]};
#pragma unroll
    for (int i = 0; i < 10; ++i) {
#pragma unroll
      for (int dl = 1; dl < 32; dl <<= 1) vals[i] += __shfl_xor_sync(0xffffffffu, vals[i], dl);
    }
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 10; ++i) s_sum[warp * 10 + i] = vals[i];
      if (quad == 0) {
        s_max[16 + 2 * half] = m_ref[0];
        s_max[16 + 2 * half + 1] = m_ref[1];
      }
    }
  }
  __syncthreads();
  // ---- partial: this thread holds dim row `tok` of O^T, columns of heads 2 * half and 2 * half + 1 ---------------------
  {
    uint32_t o[8];
    tmem_ld8(tmem_addr(tmem, my_lanes, Cfg::kColO + 8 * half), o);
    tmem_wait_ld();
    // row r of the value operand = slot r % 8 of dim group r / 8: nibble order 0, 4, 1, 5, 2, 6, 3, 7; nibbles 0, 4, 2, 6
    // sat in mantissa bits 0-3 (2^-24), the others in bits 4-7 (2^-20)
    const int r = tok;
    const int j = r & 7;
    const int nib = (j >> 1) + ((j & 1) ? 4 : 0);
    const int dim = (r & ~7) + nib;
    const float unscale = (j & 2) ? 1048576.0f : 16777216.0f;
    const int group = dim >> 5;
    const int64_t part = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity + out_slot;
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int h = 2 * half + h2;
      if (h >= g_count) continue;
      float l_all = 0.0f, z_all = 0.0f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        l_all += s_sum[(half * 4 + w) * 10 + h2];
        z_all += s_sum[(half * 4 + w) * 10 + 2 + h2 * 4 + group];
      }
      const uint32_t cell = o[h2 * 4 + group];
      const float value = steps_done > 0 ? fmaf(__uint_as_float(cell), unscale, z_all) : 0.0f;
      p.values[(part + (int64_t)h * p.chunk_capacity) * D + dim] = value;
      if (r == 0) {
        const float m = s_max[16 + h];
        float* stats_out = p.stats + (part + (int64_t)h * p.chunk_capacity) * 2;
        stats_out[0] = (steps_done > 0 && m != -INFINITY) ? m * qconst[h] * 0.6931471805599453f : -INFINITY;
        stats_out[1] = steps_done > 0 ? l_all : 0.0f;
      }
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, Cfg::kColumns);

  // The window kernel's partials and, when it arrives last, its merged output must be complete before this CTA
  // counts itself in (fused merge) or the kernel ends (two-pass merge).
  umma_wait_prior_grids();
  if (p.fused.counters != nullptr) {
    const int64_t head0 = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity;
    __syncthreads();
    fused_combine_tail<T, D, kUmmaThreads>(p.fused, b, hq0, g_count, active_chunks, p.chunk_capacity,
                                           p.stats + head0 * 2, p.values + head0 * D,
                                           reinterpret_cast<float*>(smem_raw), (int64_t)b * gridDim.y + blockIdx.y);
  }
}


template <typename T, int BITS>
static int launch_umma(const TqDecodeParams& p, int batch, cudaStream_t stream) {
  using Cfg = UmmaCfg<T, BITS>;
  auto kernel = tq_decode_umma_kernel<T, BITS>;
  static bool configured[64] = {};
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !configured[device]) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  // a page chunk is copied as one run, so it must have exactly the tile layout the kernel reads
  if (p.layout.off_kcodes != Cfg::kOffKey || p.layout.off_knorm != Cfg::kOffNorm ||
      p.layout.off_krnorm != Cfg::kOffRnorm || p.layout.off_vdata != Cfg::kOffVal ||
      p.layout.off_vscale != Cfg::kOffScale || p.layout.off_vzero != Cfg::kOffZero ||
      p.layout.chunk_bytes < Cfg::kTileDataBytes)
    return set_error(ANNA_ERR_INVALID, "packed page layout does not match the decode kernel's tile layout");
  dim3 prep_grid((unsigned)p.kv_heads, (unsigned)batch);
  tq_prepare_queries_umma_kernel<T, BITS><<<prep_grid, 128, 0, stream>>>(p);
  int rc = check_launch("tq_prepare_queries_umma_kernel");
  if (rc != ANNA_OK) return rc;
  rc = launch_tq_window_split(p, batch, kUmmaDim, std::is_same<T, __half>::value ? ANNA_DTYPE_F16 : ANNA_DTYPE_BF16,
                              stream);
  if (rc != ANNA_OK) return rc;
  if (p.num_chunks > p.num_window_chunks) {
    // programmatic dependent launch: the packed chunks run beside the (small) window launch instead of after it; the
    // query operand they read comes from the launch before that one, which has completed by then
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)p.num_chunks, (unsigned)p.kv_heads, (unsigned)batch);
    config.blockDim = dim3(kUmmaThreads);
    config.dynamicSmemBytes = Cfg::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    ANNA_CUDA_CHECK(cudaLaunchKernelEx(&config, kernel, p));
    rc = check_launch("tq_decode_umma_kernel");
  }
  return rc;
}

int tq_decode_umma_faults(int* count) {
  int32_t value = 0;
  ANNA_CUDA_CHECK(cudaMemcpyFromSymbol(&value, g_tq_umma_faults, sizeof(value)));
  *count = (int)value;
  return ANNA_OK;
}

size_t tq_umma_query_bytes() { return (size_t)UmmaCfg<__half, 4>::kQBytes; }

bool tq_split_umma_applicable(const TqDecodeParams& p, int head_dim, int bits, int dtype) {
  // Opt-in (ANNA_B200_TQ_UMMA=1, read once per process): measured slower than the mma.sync kernel so far -- with two
  // CTAs of eight warps per SM the step loop is bound by the latency of its own instruction chain, not by the tensor
  // core or by HBM.
  static const bool enabled = [] {
    const char* flag = std::getenv("ANNA_B200_TQ_UMMA");
    return flag != nullptr && flag[0] != '\0' && flag[0] != '0';
  }();
  if (!enabled) return false;
  if (dtype != ANNA_DTYPE_F16 && dtype != ANNA_DTYPE_BF16) return false;
  if (head_dim != kUmmaDim || (bits != 3 && bits != 4) || p.groups > kUmmaHeads) return false;
  if (p.value_group != 32 || p.block_size != 16 || p.chunk_tokens % kUmmaStepTokens != 0) return false;
  if (p.max_len >= (int64_t)1 << 31 || p.query_frags == nullptr) return false;
  return true;
}

int launch_tq_split_umma(const TqDecodeParams& p, int batch, int bits, int dtype, cudaStream_t stream) {
  if (dtype == ANNA_DTYPE_BF16)
    return bits == 4 ? launch_umma<__nv_bfloat16, 4>(p, batch, stream) : launch_umma<__nv_bfloat16, 3>(p, batch, stream);
  return bits == 4 ? launch_umma<__half, 4>(p, batch, stream) : launch_umma<__half, 3>(p, batch, stream);
}

}  // namespace anna
