// Tensor-core split pass of single-token GQA decode over packed TurboQuant pages (16-bit cache dtypes).
//
// A CTA (4 warps) owns one (row, kv head, chunk).  Chunks that cover the un-quantized window ring run the dense
// tensor-core body (dense_mma_body.cuh); chunks over the packed prefix run the path below.  Per warp and 16-token tile:
//
//   packed bytes of the tile --bulk copy (cp.async.bulk, mbarrier)--> shared (2 stages per warp); a tile of a 16-token
//              page is one linear copy issued by one lane, larger pages take six
//   K codes -> fp16 A fragments in registers: byte-permute (PRMT) table lookups turn 4-bit / 2-bit fields into
//              centroid values and +-1 signs, two tokens x D/4 coordinates per lane, no shared-memory round trip
//   S1[16 tok x 8 heads] = centroid(K) . Q1^T      S2 = sign(K) . Q2^T        (2 x D/16 mma.sync m16n8k16, fp16)
//   score = norm * (S1 + rnorm * S2)   with Q1 = fwht(s1*q) * scaling / sqrt(D)  (times c0 for 1-bit indices)
//                                           Q2 = fwht(s2*fwht(s1*q)) * scaling * sqrt(pi/2) / D^1.5
//   online softmax in fp32 on the C fragments; P packed to fp16 and transposed with movmatrix
//   V codes -> fp16 (magic-number trick) -> (code * scale + zero) in fp16 pairs -> A fragments of V^T
//   O^T[D x 8 heads] += V^T . P^T                                              (D/16 mma.sync)
//
// The K-dimension slots of the two score products are free to permute, so each lane takes the coordinates whose
// codes it can unpack with the fewest instructions; Q1 / Q2 fragments are gathered with the same permutation.
#include "dense_mma_body.cuh"
#include "mbarrier_utils.cuh"
#include "tq_common.cuh"
#include "prefill_params.cuh"
#include "tq_decode_params.cuh"

#include <cstdlib>

namespace anna {

__device__ int32_t g_tq_mma_faults;  // bumped when a bounded wait on a tile copy expires

// Byte permute and logic helpers are plain intrinsics / C so that the compiler can fold the constant selectors and
// masks into immediates; the packed fp16 arithmetic goes through PTX on raw registers.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t bits) { return (x & mask) | bits; }
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// Packed fp16 fused multiply-add on raw registers.  (Going through __half2 objects costs a logic operation per call to
// put the two halves back together.)
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// A value the compiler cannot see through: `lane` rides along as an unused operand so that the result counts as
// different in every lane and stays in an ordinary register.  (A value known to be the same in all lanes is moved to a
// uniform register when registers are short and copied back, one instruction each time, in front of every use that
// cannot read it from there.)
__device__ __forceinline__ uint32_t pinned_u32(uint32_t value, int lane) {
  uint32_t r;
  asm volatile("{\n .reg .b32 t;\n mov.b32 t, %2;\n mov.b32 %0, %1;\n}\n" : "=r"(r) : "r"(value), "r"(lane));
  return r;
}
// (x & mask) | bits as one three-input logic operation on registers (written out in C with two register constants it
// becomes two instructions).
__device__ __forceinline__ uint32_t and_or_regs(uint32_t x, uint32_t mask, uint32_t bits) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(x), "r"(mask), "r"(bits));
  return r;
}

// fp16 pair (+-1, +-1) from bits b and b + 16 of x (0 <= b <= 15): a set bit gives +1.  One shift and one logic op,
// ((x << (15 - b)) & 0x80008000) ^ 0xBC00BC00 with both constants in registers (`sign_bits`, `minus_one`).
__device__ __forceinline__ uint32_t pm_one_pair(uint32_t x, int b, uint32_t sign_bits, uint32_t minus_one) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;\n" : "=r"(r) : "r"(x << (15 - b)), "r"(sign_bits), "r"(minus_one));
  return r;
}
// mma.sync m16n8k16 (fp16 in, fp32 accumulate) without the volatile qualifier: a pure function of its operands, so
// the compiler may interleave the independent accumulation chains of this kernel
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// mma.sync m16n8k32 (signed 8-bit in, 32-bit integer accumulate); same C fragment layout as the fp16 shape above
__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Byte permute in PTX's default mode: result byte i is the byte of {a (0-3), b (4-7)} that bits 0-2 of nibble i of
// the low half of `sel` name, or, when bit 3 of that nibble is set, eight copies of that byte's top bit.
__device__ __forceinline__ uint32_t prmt_ptx(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// N consecutive 32-bit words from shared memory with the widest aligned load (the address is N*4-byte aligned).
template <int N>
__device__ __forceinline__ void lds_words(const uint8_t* ptr, uint32_t (&dst)[N]) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const uint4 v = reinterpret_cast<const uint4*>(ptr)[i];
      dst[4 * i] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
    }
  } else if constexpr (N == 2) {
    const uint2 v = *reinterpret_cast<const uint2*>(ptr);
    dst[0] = v.x; dst[1] = v.y;
  } else {
    static_assert(N == 1, "unsupported word count");
    dst[0] = *reinterpret_cast<const uint32_t*>(ptr);
  }
}

// Blocks until the grids this one was launched behind (programmatic stream serialization) have completed and their
// writes are visible; returns at once for a normal launch.  Every CTA of the packed kernel passes through it before
// it exits, so "the packed kernel is done" implies "the window kernel is done" for whatever comes next in the stream.
__device__ __forceinline__ void wait_for_prior_grids() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#ifndef ANNA_TQ_CTAS128
#define ANNA_TQ_CTAS128 4
#endif
#ifndef ANNA_TQ_CTAS256
#define ANNA_TQ_CTAS256 3
#endif
#ifndef ANNA_TQ_TILES_PER_STEP
#define ANNA_TQ_TILES_PER_STEP 2
#endif
#ifndef ANNA_TQ_RING_TILES
#define ANNA_TQ_RING_TILES 4
#endif
#ifndef ANNA_TQ_FINE_QUERY
#define ANNA_TQ_FINE_QUERY 1
#endif
#ifndef ANNA_TQ_OVERLAP_WINDOW
#define ANNA_TQ_OVERLAP_WINDOW 1
#endif
constexpr float kLazyRescale = 8.0f;  // log2 units: probabilities stay below 2^8, well inside fp16

template <typename T, int D, int BITS>
struct TqMmaCfg {
  static constexpr int kSteps = D / 16;
  // 4-bit key codes are scored as 8-bit integers: one byte permute turns four codes into four centroid bytes, another
  // into four sign bytes, and the rotated queries are rounded to 8 bits per head (127 steps up to their largest
  // coordinate) -- about a third of the instructions of the fp16 expansion the 2- and 3-bit formats use
  static constexpr bool kInt8Keys = BITS == 4;
  static constexpr int kSteps8 = D / 32;                       // k-steps of the 8-bit score products
  static constexpr int kFragBytes = kInt8Keys ? 32 * kSteps8 * 16 : 32 * kSteps * 16;  // query fragments of one unit
  static constexpr int kFragLoBytes = kInt8Keys ? 32 * kSteps8 * 8 : 0;  // second (fine) byte of the rotated queries
  static constexpr int kConstOffset = kFragBytes + kFragLoBytes;         // per-head factors and the centroid bytes
  static_assert(!kInt8Keys || kConstOffset + 128 <= 32 * D, "the query scratch of a unit is 32 * D bytes");
  static constexpr int kGroups = D / 32;                       // value group size is 32 on this path
  static constexpr int kKeyBytes = D * BITS / 8;               // packed key bytes per token
  static constexpr int kIdxBytes = BITS == 3 ? D / 4 : kKeyBytes;  // first plane (all of it unless BITS == 3)
  static constexpr int kSignBytes = BITS == 3 ? D / 8 : 0;     // separate sign plane of the 3-bit format
  static constexpr int kValBytes = D / (BITS == 2 ? 4 : 2);
  // stage layout (bytes): the layout of a 16-token chunk, so a tile of a 16-token page is one linear copy
  static constexpr int kOffKey = 0;
  static constexpr int kOffNorm = 16 * kKeyBytes;
  static constexpr int kOffRnorm = kOffNorm + 64;
  static constexpr int kOffVal = kOffRnorm + 64;
  static constexpr int kOffScale = kOffVal + 16 * kValBytes;
  static constexpr int kOffZero = kOffScale + 16 * kGroups * 2;
  static constexpr int kStageBytes = (kOffZero + 16 * kGroups * 2 + 127) / 128 * 128;
  static constexpr int kTilesPerStep = ANNA_TQ_TILES_PER_STEP;  // 16-token tiles a warp scores together (one softmax update)
  static constexpr int kStages = ANNA_TQ_RING_TILES / kTilesPerStep;  // steps per warp ring; kStages - 1 are in flight
  static constexpr int kMinBlocks = D >= 256 ? ANNA_TQ_CTAS256 : ANNA_TQ_CTAS128;
  static constexpr int kWarpSmem = kStages * kTilesPerStep * kStageBytes;
  static constexpr int kPackedSmem = kMmaWarps * kWarpSmem;
  static constexpr int kMergeSmem = (2 * kMmaWarps * 8 + kMmaWarps * 8 * (D + 4)) * 4;
  static constexpr int kTailSmem = 8 * kFusedMaxChunks * 4;
  static constexpr int kSmemBytes0 = kPackedSmem > kMergeSmem ? kPackedSmem : kMergeSmem;
  static constexpr int kWorkSmem = ((kSmemBytes0 > kTailSmem ? kSmemBytes0 : kTailSmem) + 15) / 16 * 16;
  // behind the working area (which the epilogue reuses): one mbarrier per warp and stage, one valid-token count per tile
  static constexpr int kBarrierBytes = kMmaWarps * kStages * 8;
  static constexpr int kQueryOffset = (kWorkSmem + kBarrierBytes + kMmaWarps * kStages * kTilesPerStep * 4 + 15) / 16 * 16;
  // 8-bit scoring keeps the query fragments of the CTA in shared memory (a 16-byte and an 8-byte load per k-step
  // and step) instead of 24 registers per lane
  static constexpr int kSmemBytes = kQueryOffset + (kInt8Keys ? kFragBytes + kFragLoBytes : 0);
  // bytes of one 16-token tile in the stage (= in a 16-token page chunk, padding excluded)
  static constexpr int kTileDataBytes = kOffZero + 16 * kGroups * 2;
  // per-lane key code words per token (this lane's D/4 coordinates)
  static constexpr int kIdxWords = BITS == 4 ? D / 32 : D / 64;
  static constexpr int kSignWords = BITS == 3 ? D / 128 : 0;
  static constexpr int kValWords = BITS == 2 ? D / 128 : D / 64;  // per token, this lane's D/8 dims
  static_assert(D == 128 || D == 256, "tensor-core TurboQuant decode is built for head_dim 128 and 256");
};

// Coordinate that lane `tig` feeds into slot k (0..3 = 2tig, 2tig+1, 2tig+8, 2tig+9) of k-step s.
template <int D, int BITS>
__device__ __forceinline__ int idx_coord(int tig, int s, int k) {
  constexpr int kRun = D / 4;
  if constexpr (BITS == 4) return tig * kRun + 4 * s + k;
  if constexpr (BITS == 3) return tig * kRun + 8 * (s / 2) + 2 * k + (s % 2);
  // 1-bit indices: bits 2c of a 16-coordinate word; a register pairs coordinates c and c + 8
  return tig * kRun + 16 * (s / 4) + 2 * (s % 4) + (k >> 1) + 8 * (k & 1);
}
template <int D, int BITS>
__device__ __forceinline__ int sign_coord(int tig, int s, int k) {
  constexpr int kRun = D / 4;
  // the two halves of a register take sign bits 16 apart in their word: 4 coordinates (4-bit codes), 8 (2-bit codes)
  // or 16 (the separate sign plane of 3-bit codes) apart
  if constexpr (BITS == 4) return tig * kRun + 8 * (s / 2) + 2 * (s % 2) + (k >> 1) + 4 * (k & 1);
  if constexpr (BITS == 3) return tig * kRun + 32 * (s / 8) + 2 * (s % 8) + (k >> 1) + 16 * (k & 1);
  return idx_coord<D, BITS>(tig, s, k);
}

// Rotates the queries of one (row, kv-head group) and stores them as fp16 B fragments in the register order of the
// split kernel: [row][group][lane][step][q1 b0, q1 b1, q2 b0, q2 b1].  Q1 = fwht(s1*q) / sqrt(D), Q2 = fwht(s2*fwht(s1*q)) / D.
template <typename T, int D, int BITS>
__global__ void __launch_bounds__(kMmaThreads) tq_prepare_queries_kernel(const TqDecodeParams p) {
  using Cfg = TqMmaCfg<T, D, BITS>;
  constexpr int E = D / 32;
  constexpr int kSteps = D / 16;
  __shared__ float q_rot[2][8][D];
  __shared__ float q_amax[2][8];
  const int group_tiles = (p.groups + 7) / 8;
  const int kvh = blockIdx.x / group_tiles;
  const int g0 = (blockIdx.x % group_tiles) * 8;
  const int g_count = min(8, p.groups - g0);
  const int b = blockIdx.y;
  const int hq0 = kvh * p.groups + g0;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const T* q_ptr = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b;
  for (int g = warp; g < 8; g += kMmaWarps) {
    float w[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int d = lane * E + j;
      w[j] = g < g_count ? ElemTraits<T>::to_float(q_ptr[(int64_t)(hq0 + g) * p.q_stride_h + d]) : 0.0f;
      if (p.signs1[d] < 0.0f) w[j] = -w[j];
    }
    warp_fwht<E>(w, lane);
    float amax1 = 0.0f, amax2 = 0.0f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int d = lane * E + j;
      q_rot[0][g][d] = w[j];
      amax1 = fmaxf(amax1, fabsf(w[j]));
      if (p.signs2[d] < 0.0f) w[j] = -w[j];
    }
    warp_fwht<E>(w, lane);
#pragma unroll
    for (int j = 0; j < E; ++j) {
      q_rot[1][g][lane * E + j] = w[j];
      amax2 = fmaxf(amax2, fabsf(w[j]));
    }
#pragma unroll
    for (int dl = 1; dl < 32; dl <<= 1) {
      amax1 = fmaxf(amax1, __shfl_xor_sync(0xffffffffu, amax1, dl));
      amax2 = fmaxf(amax2, __shfl_xor_sync(0xffffffffu, amax2, dl));
    }
    if (lane == 0) {
      q_amax[0][g] = amax1;
      q_amax[1][g] = amax2;
    }
  }
  __syncthreads();
  // score (log2 units) = norm * (S1 + rnorm * S2) with every constant folded into the fragments:
  //   q.k_hat = norm/D * [Q1.c + sqrt(pi/2)/sqrt(D) * rnorm * Q2.sign],  Q1 = fwht(s1*q), Q2 = fwht(s2*Q1)
  //   (1-bit indices: the centroids are +-c0 and the fragments carry +-1, so c0 goes into the factor)
  const float inv_sqrt_d = rsqrt_dim_const<D>();
  const float log2e = 1.4426950408889634f;
  const float f1 = (BITS == 2 ? __ldg(p.centroids + 1) : 1.0f) * p.scaling * log2e * inv_sqrt_d * inv_sqrt_d;
  const float f2 = p.scaling * log2e * 1.2533141373155001f * inv_sqrt_d * inv_sqrt_d * inv_sqrt_d;
  // every unit owns 32 * D bytes of the scratch
  uint8_t* unit = reinterpret_cast<uint8_t*>(p.query_frags) + ((int64_t)b * gridDim.x + blockIdx.x) * (32 * D);
  if constexpr (Cfg::kInt8Keys) {
    // 8-bit B fragments of m16n8k32: lane (gid, tig) feeds head gid with the coordinates of its code word s,
    // tig * D/4 + 8s + {0..3} in the first register and + {4..7} in the second.  The rotated query is split into a
    // coarse byte (127 steps up to the head's largest coordinate) and a fine byte (the rounding remainder in 1/254
    // steps), so the centroid product sees about 15 bits of it; the sign product uses a coarse byte only.
    //   [s][lane][q1 b0, q1 b1, q2 b0, q2 b1]   then   [s][lane][q1 fine b0, q1 fine b1]
    // Behind them, per head: the factor of the centroid product, the factor of the sign product and the integer the
    // sign accumulators start from (sign bytes are 2 for a clear bit and 0 for a set one: 2 * sum over clear bits
    // minus the sum over all coordinates is minus the +-1 product); then the centroids as signed bytes.
    constexpr int kSteps8 = Cfg::kSteps8;
    constexpr int kEntries = 1 << (BITS - 1);
    __shared__ float cent_scale;
    if (warp == 0) {
      // The byte scale of the centroids is the one, among 256 candidates from 127 down to 63 steps for the largest
      // centroid, that leaves the smallest squared rounding error over the codebook.
      float cent[kEntries], cmax = 0.0f;
#pragma unroll
      for (int e = 0; e < kEntries; ++e) {
        cent[e] = __ldg(p.centroids + e);
        cmax = fmaxf(cmax, fabsf(cent[e]));
      }
      float best_err = INFINITY, best_k = 0.0f;
      if (cmax > 0.0f) {
        for (int j = lane; j < 256; j += 32) {
          const float k = (127.0f - 0.25f * (float)j) / cmax;
          float err = 0.0f;
#pragma unroll
          for (int e = 0; e < kEntries; ++e) {
            const float d = (cent[e] * k - rintf(cent[e] * k)) / k;
            err += d * d;
          }
          if (err < best_err) { best_err = err; best_k = k; }
        }
      }
#pragma unroll
      for (int dl = 1; dl < 32; dl <<= 1) {
        const float other_err = __shfl_xor_sync(0xffffffffu, best_err, dl);
        const float other_k = __shfl_xor_sync(0xffffffffu, best_k, dl);
        if (other_err < best_err || (other_err == best_err && other_k > best_k)) { best_err = other_err; best_k = other_k; }
      }
      if (lane == 0) {
        cent_scale = best_k;
        uint32_t lut[2] = {0u, 0u};
#pragma unroll
        for (int e = 0; e < kEntries; ++e)
          lut[e / 4] |= ((uint32_t)__float2int_rn(cent[e] * best_k) & 0xffu) << (8 * (e % 4));
        uint32_t* consts = reinterpret_cast<uint32_t*>(unit + Cfg::kConstOffset);
        consts[24] = lut[0];
        consts[25] = lut[1];
      }
    }
    __syncthreads();
    auto coarse = [](float v, float k) { return max(-127, min(127, __float2int_rn(v * k))); };
    auto fine = [](float v, float k, int c) { return max(-127, min(127, __float2int_rn((v * k - (float)c) * 254.0f))); };
    uint4* out = reinterpret_cast<uint4*>(unit);
    uint2* out_lo = reinterpret_cast<uint2*>(unit + Cfg::kFragBytes);
    for (int item = threadIdx.x; item < 32 * kSteps8; item += kMmaThreads) {
      const int ln = item / kSteps8;
      const int s = item % kSteps8;
      const int gid = ln >> 2, tig = ln & 3;
      const float k1 = q_amax[0][gid] > 0.0f ? 127.0f / q_amax[0][gid] : 0.0f;
      const float k2 = q_amax[1][gid] > 0.0f ? 127.0f / q_amax[1][gid] : 0.0f;
      const float* r1 = q_rot[0][gid] + tig * (D / 4) + 8 * s;
      const float* r2 = q_rot[1][gid] + tig * (D / 4) + 8 * s;
      uint32_t w[4] = {0u, 0u, 0u, 0u}, wl[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c0 = coarse(r1[i], k1), c1 = coarse(r1[4 + i], k1);
        w[0] |= ((uint32_t)c0 & 0xffu) << (8 * i);
        w[1] |= ((uint32_t)c1 & 0xffu) << (8 * i);
        wl[0] |= ((uint32_t)fine(r1[i], k1, c0) & 0xffu) << (8 * i);
        wl[1] |= ((uint32_t)fine(r1[4 + i], k1, c1) & 0xffu) << (8 * i);
        w[2] |= ((uint32_t)coarse(r2[i], k2) & 0xffu) << (8 * i);
        w[3] |= ((uint32_t)coarse(r2[4 + i], k2) & 0xffu) << (8 * i);
      }
      out[s * 32 + ln] = make_uint4(w[0], w[1], w[2], w[3]);
      out_lo[s * 32 + ln] = make_uint2(wl[0], wl[1]);
    }
    if (threadIdx.x < 8) {
      const int g = threadIdx.x;
      const float k2 = q_amax[1][g] > 0.0f ? 127.0f / q_amax[1][g] : 0.0f;
      int total = 0;
      for (int d = 0; d < D; ++d) total += coarse(q_rot[1][g][d], k2);
      float* consts = reinterpret_cast<float*>(unit + Cfg::kConstOffset);
      consts[g] = cent_scale > 0.0f ? (q_amax[0][g] * f1 / 127.0f) / cent_scale / (ANNA_TQ_FINE_QUERY ? 254.0f : 1.0f) : 0.0f;
      consts[8 + g] = -(q_amax[1][g] * f2 / 127.0f);
      reinterpret_cast<int*>(consts)[16 + g] = -total;
    }
  } else {
    uint4* out = reinterpret_cast<uint4*>(unit);
    for (int item = threadIdx.x; item < 32 * kSteps; item += kMmaThreads) {
      const int ln = item / kSteps;
      const int s = item % kSteps;
      const int gid = ln >> 2, tig = ln & 3;
      const float* r1 = q_rot[0][gid];
      const float* r2 = q_rot[1][gid];
      uint4 v;
      v.x = pack2<__half>(r1[idx_coord<D, BITS>(tig, s, 0)] * f1, r1[idx_coord<D, BITS>(tig, s, 1)] * f1);
      v.y = pack2<__half>(r1[idx_coord<D, BITS>(tig, s, 2)] * f1, r1[idx_coord<D, BITS>(tig, s, 3)] * f1);
      v.z = pack2<__half>(r2[sign_coord<D, BITS>(tig, s, 0)] * f2, r2[sign_coord<D, BITS>(tig, s, 1)] * f2);
      v.w = pack2<__half>(r2[sign_coord<D, BITS>(tig, s, 2)] * f2, r2[sign_coord<D, BITS>(tig, s, 3)] * f2);
      out[item] = v;
    }
  }
}

// Split pass over the un-quantized window ring of every row: the dense tensor-core body with ring addressing.
// Grid (num_window_chunks, kv_heads * group tiles, batch).  Also writes the zero output of empty rows.
template <typename T, int D>
__global__ void __launch_bounds__(kMmaThreads, MmaCfg<D>::kMinBlocks) tq_window_split_mma_kernel(const TqDecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
#if ANNA_TQ_OVERLAP_WINDOW
  // The packed-chunk kernel that follows in the stream reads nothing this kernel writes before the arrival counters
  // say so, and each of its CTAs waits for this grid to complete before it counts itself in or exits, so it may start
  // as soon as every CTA here has been scheduled.
  asm volatile("griddepcontrol.launch_dependents;\n" ::);
#endif
  const int slot = blockIdx.x;
  const int group_tiles = (p.groups + 7) / 8;
  const int kvh = blockIdx.y / group_tiles;
  const int g0 = (blockIdx.y % group_tiles) * 8;
  const int g_count = min(8, p.groups - g0);
  const int b = blockIdx.z;
  const int hq0 = kvh * p.groups + g0;
  int64_t len64 = p.lengths[b];
  len64 = max((int64_t)0, min(len64, p.max_len));
  const int len = (int)len64;
  const int R = p.residual_len;
  const int Lq = len > R ? len - R : 0;
  const int active_window = (len - Lq + p.chunk_tokens - 1) / p.chunk_tokens;
  const int active_chunks = active_window + (Lq + p.chunk_tokens - 1) / p.chunk_tokens;
  if (len == 0) {
    if (p.fused.counters != nullptr && slot == 0) fused_write_zero_row<T, D, kMmaThreads>(p.fused, b, hq0, g_count);
    return;
  }
  if (slot >= active_window) return;
  DenseDecodeParams dp{};
  dp.q = p.q; dp.q_stride_b = p.q_stride_b; dp.q_stride_h = p.q_stride_h;
  const int64_t ring_elems = (int64_t)R * D;
  const int64_t slot_base = p.window_slots[b] * 2 * p.kv_heads * ring_elems;
  dp.key = reinterpret_cast<const T*>(p.window) + slot_base;
  dp.value = reinterpret_cast<const T*>(p.window) + slot_base + (int64_t)p.kv_heads * ring_elems;
  dp.page_table = nullptr;
  dp.kv_stride_b = 0; dp.kv_stride_h = ring_elems; dp.kv_stride_t = D;
  dp.ring_len = R;
  dp.block_size = 1; dp.block_shift = 0;
  dp.stats = p.stats; dp.values = p.values;
  dp.q_heads = p.q_heads; dp.kv_heads = p.kv_heads; dp.groups = p.groups;
  dp.chunk_tokens = p.chunk_tokens; dp.num_chunks = p.num_chunks; dp.chunk_capacity = p.chunk_capacity;
  dp.scaling = p.scaling;
  dp.fused = p.fused;
  const int t0 = Lq + slot * p.chunk_tokens;
  const int t1 = min(len, t0 + p.chunk_tokens);
  dense_split_mma_body<T, D>(dp, smem_raw, b, kvh, g0, g_count, t0, t1, slot, active_chunks,
                             (int64_t)b * gridDim.y + blockIdx.y);
}

template <typename T, int D, int BITS>
__global__ void __launch_bounds__(kMmaThreads, TqMmaCfg<T, D, BITS>::kMinBlocks)
    tq_decode_split_mma_kernel(const TqDecodeParams p) {
  using Cfg = TqMmaCfg<T, D, BITS>;
  constexpr int U = Cfg::kTilesPerStep;
  extern __shared__ __align__(1024) uint8_t smem_raw[];

  const int slot = blockIdx.x;
  const int group_tiles = (p.groups + 7) / 8;
  const int kvh = blockIdx.y / group_tiles;
  const int g0 = (blockIdx.y % group_tiles) * 8;
  const int g_count = min(8, p.groups - g0);
  const int b = blockIdx.z;
  const int hq0 = kvh * p.groups + g0;

  int64_t len64 = p.lengths[b];
  len64 = max((int64_t)0, min(len64, p.max_len));
  const int len = (int)len64;
  const int R = p.residual_len;
  const int Lq = len > R ? len - R : 0;
  const int win = len - Lq;
  const int active_window = (win + p.chunk_tokens - 1) / p.chunk_tokens;
  const int active_packed = (Lq + p.chunk_tokens - 1) / p.chunk_tokens;
  const int active_chunks = active_window + active_packed;
  if (len == 0 || slot < p.num_window_chunks) {  // window chunks run in tq_window_split_mma_kernel
    wait_for_prior_grids();
    return;
  }

  // ---- packed chunks ------------------------------------------------------------------------------------------------------
  const int chunk = slot - p.num_window_chunks;
  const int t0 = chunk * p.chunk_tokens;
  if (t0 >= Lq) {
    wait_for_prior_grids();
    return;
  }
  const int t1 = min(Lq, t0 + p.chunk_tokens);
  const int out_slot = active_window + chunk;  // active slots stay contiguous: [window | packed]
  const int num_tiles = (t1 - t0 + kTileTokens - 1) / kTileTokens;
  if (threadIdx.x == 0) {
    const uint32_t bars = smem_u32(smem_raw + Cfg::kWorkSmem);
    for (int i = 0; i < kMmaWarps * Cfg::kStages; ++i) mbar_init(bars + i * 8, 1);
    mbar_init_fence();
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2;
  const int tig = lane & 3;
  // Q fragments (softmax scale and log2(e) folded in) were prepared by tq_prepare_queries_kernel in exactly this
  // lane's register order: [row b][blockIdx.y][lane][step][q1 b0, q1 b1, q2 b0, q2 b1]; fp16 pairs, or bytes with the
  // per-head factors behind them when the key codes are scored as 8-bit integers
  constexpr int kQSteps = Cfg::kInt8Keys ? 1 : Cfg::kSteps;
  uint32_t q1f[kQSteps][2], q2f[kQSteps][2];
  float beta1[2] = {0.0f, 0.0f}, beta2[2] = {0.0f, 0.0f};  // this lane's two heads (columns 2tig, 2tig + 1)
  int s2_start[2] = {0, 0};
  uint32_t cent_bytes[2] = {0u, 0u};
  const uint4* q_coarse = reinterpret_cast<const uint4*>(smem_raw + Cfg::kQueryOffset) + lane;          // [s][lane]
  const uint2* q_fine = reinterpret_cast<const uint2*>(smem_raw + Cfg::kQueryOffset + Cfg::kFragBytes) + lane;
  {
    const uint8_t* unit = reinterpret_cast<const uint8_t*>(p.query_frags) + ((int64_t)b * gridDim.y + blockIdx.y) * (32 * D);
    if constexpr (Cfg::kInt8Keys) {
      // the CTA's query fragments go to shared memory once; every warp reads them after the barrier below
      const uint4* src = reinterpret_cast<const uint4*>(unit);
      uint4* dst = reinterpret_cast<uint4*>(smem_raw + Cfg::kQueryOffset);
      for (int i = threadIdx.x; i < (Cfg::kFragBytes + Cfg::kFragLoBytes) / 16; i += kMmaThreads) dst[i] = __ldg(src + i);
      const float* consts = reinterpret_cast<const float*>(unit + Cfg::kConstOffset);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        beta1[c] = __ldg(consts + 2 * tig + c);
        beta2[c] = __ldg(consts + 8 + 2 * tig + c);
        s2_start[c] = __ldg(reinterpret_cast<const int*>(consts) + 16 + 2 * tig + c);
      }
      cent_bytes[0] = __ldg(reinterpret_cast<const uint32_t*>(consts) + 24);
      cent_bytes[1] = __ldg(reinterpret_cast<const uint32_t*>(consts) + 25);
      __syncthreads();
    } else {
      const uint4* frag = reinterpret_cast<const uint4*>(unit) + lane * kQSteps;
#pragma unroll
      for (int s = 0; s < kQSteps; ++s) {
        const uint4 v = __ldg(frag + s);
        q1f[s][0] = v.x; q1f[s][1] = v.y; q2f[s][0] = v.z; q2f[s][1] = v.w;
      }
    }
  }

  // centroid lookup tables for PRMT (up to 8 entries): low bytes and high bytes of the fp16 centroids, or -- 4-bit
  // codes -- the centroids as signed bytes in lut_lo, as the query preparation rounded them
  uint32_t lut_lo[2] = {0u, 0u}, lut_hi[2] = {0u, 0u};
  if constexpr (Cfg::kInt8Keys) {
    lut_lo[0] = pinned_u32(cent_bytes[0], lane);
    lut_lo[1] = pinned_u32(cent_bytes[1], lane);
  } else if constexpr (BITS != 2) {
    constexpr int kEntries = 1 << (BITS - 1);
#pragma unroll
    for (int e = 0; e < kEntries; ++e) {
      const __half h = __float2half_rn(__ldg(p.centroids + e));
      const uint32_t bits = (uint32_t)__half_as_ushort(h);
      lut_lo[e / 4] |= (bits & 0xffu) << (8 * (e % 4));
      lut_hi[e / 4] |= (bits >> 8) << (8 * (e % 4));
    }
    if constexpr (BITS == 3) {  // 4 entries: mirror them so that PRMT may pick from either operand
      lut_lo[1] = lut_lo[0];
      lut_hi[1] = lut_hi[0];
    }
  }

  // loop constants held in registers
  // (only the ones this instantiation uses are created)
  const uint32_t nib_mask = BITS != 2 ? pinned_u32(0x03C003C0u, lane) : 0u;    // 4-bit value codes
  const uint32_t magic16 = BITS != 2 ? pinned_u32(0x4C004C00u, lane) : 0u;
  const uint32_t kTwo = BITS == 4 ? pinned_u32(0x02020202u, lane) : 0u;        // 4-bit key codes
  const uint32_t kIdxMask = BITS == 4 ? pinned_u32(0x77777777u, lane) : 0u;
  const uint32_t kSignBits = BITS != 4 ? pinned_u32(0x80008000u, lane) : 0u;   // +-1 fragments of 2- and 3-bit key codes
  const uint32_t kMinusOne = BITS != 4 ? pinned_u32(0xBC00BC00u, lane) : 0u;
  const uint32_t kTwoBitMask = BITS == 2 ? pinned_u32(0x03000300u, lane) : 0u;  // 2-bit value codes
  const uint32_t kMagic4 = BITS == 2 ? pinned_u32(0x44004400u, lane) : 0u;
  (void)nib_mask; (void)magic16; (void)kTwo; (void)kIdxMask; (void)kSignBits; (void)kMinusOne; (void)kTwoBitMask;
  (void)kMagic4;

  const uint32_t warp_smem_u32 = smem_u32(smem_raw + warp * Cfg::kWarpSmem);
  const uint8_t* warp_smem = smem_raw + warp * Cfg::kWarpSmem;
  const int32_t* table_row = p.block_table + (int64_t)b * p.table_stride;
  const uint32_t block_size = (uint32_t)p.block_size;
  const int block_shift = p.block_shift;
  const uint32_t bars_u32 = smem_u32(smem_raw + Cfg::kWorkSmem) + warp * Cfg::kStages * 8;
  volatile int* stage_valid = reinterpret_cast<volatile int*>(smem_raw + Cfg::kWorkSmem + Cfg::kBarrierBytes) +
                              warp * Cfg::kStages * U;
  // Start the copies of one step (U consecutive 16-token tiles) into a stage.  Each tile slot of the stage has the
  // layout of a 16-token page chunk, so with 16-token pages a tile is one linear run; with larger pages it is six runs
  // (codes, norms, residual norms, value codes, scales, zeros).  Lanes 0 .. U-1 look up and copy one tile each; lane 0
  // arms the stage's mbarrier with the bytes of all of them first.  Called by the whole warp.
  auto issue_step = [&](int step, int stage) {
    int valid = 0;
    const uint8_t* chunk_ptr = nullptr;
    int s0 = 0;
    if (lane < U) {
      const int tile = (warp + step * kMmaWarps) * U + lane;
      if (tile < num_tiles) {
        const int ts = t0 + tile * kTileTokens;
        const uint32_t blk = block_shift >= 0 ? ((uint32_t)ts >> block_shift) : ((uint32_t)ts / block_size);
        s0 = ts - (int)(blk * block_size);  // first slot of the tile inside its page
        const int32_t pid = table_row[blk];
        if (pid >= 0 && pid < p.num_pages) {  // else a hole in the block table: nothing to copy
          valid = min(kTileTokens, t1 - ts);
          chunk_ptr = p.pages + ((int64_t)pid * p.kv_heads + kvh) * p.layout.chunk_bytes;
        }
      }
      stage_valid[stage * U + lane] = valid;
    }
    const uint32_t bar = bars_u32 + stage * 8;
    const unsigned have = __ballot_sync(0xffffffffu, valid > 0);
    if (lane == 0) {
      if (have != 0u) mbar_expect_tx(bar, (uint32_t)__popc(have) * Cfg::kTileDataBytes);
      else mbar_arrive(bar);  // the phase completes at once
    }
    __syncwarp();
    if (valid > 0) {
      const uint32_t dst = warp_smem_u32 + (stage * U + lane) * Cfg::kStageBytes;
      if (block_size == (uint32_t)kTileTokens) {
        bulk_copy_g2s(dst, chunk_ptr, Cfg::kTileDataBytes, bar);
      } else {
        bulk_copy_g2s(dst + Cfg::kOffKey, chunk_ptr + p.layout.off_kcodes + s0 * Cfg::kKeyBytes, 16 * Cfg::kKeyBytes, bar);
        bulk_copy_g2s(dst + Cfg::kOffNorm, chunk_ptr + p.layout.off_knorm + 4 * s0, 64, bar);
        bulk_copy_g2s(dst + Cfg::kOffRnorm, chunk_ptr + p.layout.off_krnorm + 4 * s0, 64, bar);
        bulk_copy_g2s(dst + Cfg::kOffVal, chunk_ptr + p.layout.off_vdata + s0 * Cfg::kValBytes, 16 * Cfg::kValBytes, bar);
        bulk_copy_g2s(dst + Cfg::kOffScale, chunk_ptr + p.layout.off_vscale + s0 * Cfg::kGroups * 2, 16 * Cfg::kGroups * 2,
                      bar);
        bulk_copy_g2s(dst + Cfg::kOffZero, chunk_ptr + p.layout.off_vzero + s0 * Cfg::kGroups * 2, 16 * Cfg::kGroups * 2,
                      bar);
      }
    }
  };

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  float o_acc[Cfg::kSteps][4];
#pragma unroll
  for (int j = 0; j < Cfg::kSteps; ++j)
#pragma unroll
    for (int r = 0; r < 4; ++r) o_acc[j][r] = 0.0f;

  const int num_steps = (num_tiles + U - 1) / U;
  const int my_steps = num_steps > warp ? (num_steps - warp + kMmaWarps - 1) / kMmaWarps : 0;
#pragma unroll
  for (int i = 0; i < Cfg::kStages - 1; ++i)
    if (i < my_steps) issue_step(i, i);

  // MMA row r of a tile holds token r ^ ((r >> 1) & 1): neighbouring token rows sit in different halves of the
  // shared-memory banks, and with this order the four token rows one value load touches fall into both halves.
  const int tok_lo = gid ^ ((gid >> 1) & 1);  // rows gid and gid + 8 of the score product
  const int tok_hi = tok_lo + 8;
  // k-slots 2tig, 2tig+1 (and +8) of the value product = the same rows
  const int tok_a0 = (2 * tig) ^ (tig & 1), tok_a1 = (2 * tig + 1) ^ (tig & 1);
  // this lane's value dims: D/8 consecutive dims starting at gid * D/8, all inside value group (gid * D/8) / 32
  const int v_group = (gid * (D / 8)) / 32;

  int stage = 0;        // stage of step n
  uint32_t phase = 0;   // parity of the mbarrier phase that step n completes
  for (int n = 0; n < my_steps; ++n) {
    __syncwarp();  // every lane is done with the stage that is re-armed next (the one step n - 1 used)
    {
      const int ahead = n + Cfg::kStages - 1;
      if (ahead < my_steps) issue_step(ahead, stage == 0 ? Cfg::kStages - 1 : stage - 1);
    }
    if (!mbar_wait(bars_u32 + stage * 8, phase)) {
      if (lane == 0) atomicAdd(&g_tq_mma_faults, 1);
      // wait (bounded) for the copies still in flight before the epilogue reuses the stages
      for (int k = 1; k < Cfg::kStages && n + k < my_steps; ++k) {
        const int st_k = (stage + k) % Cfg::kStages;
        (void)mbar_wait(bars_u32 + st_k * 8, (uint32_t)((n + k) / Cfg::kStages) & 1u);
      }
      break;  // give up on this chunk: the fault counter tells the host that the output is not valid
    }
    const int cur = stage;
    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
    int valid[U];
    int valid_sum = 0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      valid[u] = stage_valid[cur * U + u];
      valid_sum += valid[u];
    }
    if (valid_sum == 0) continue;  // holes only: no token of this step exists
    const bool full = valid_sum == U * kTileTokens;
    const uint8_t* st0 = warp_smem + cur * U * Cfg::kStageBytes;

    // ---- scores: U independent pairs of accumulation chains ------------------------------------------------------------
    float s1[U][4], s2[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < 4; ++r) s1[u][r] = s2[u][r] = 0.0f;
    {
      uint32_t iw_lo[U][Cfg::kIdxWords], iw_hi[U][Cfg::kIdxWords];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint8_t* keys = st0 + u * Cfg::kStageBytes + Cfg::kOffKey + tig * (Cfg::kIdxWords * 4);
        lds_words<Cfg::kIdxWords>(keys + tok_lo * Cfg::kKeyBytes, iw_lo[u]);
        lds_words<Cfg::kIdxWords>(keys + tok_hi * Cfg::kKeyBytes, iw_hi[u]);
      }
      if constexpr (BITS == 4) {
        // one code word = 8 coordinates of a token = one k-step: its low half-word selects four centroid bytes (and,
        // unmasked, four sign bytes: bit 3 of a selector nibble asks for the top bit of the byte 0x02, i.e. 0), its high
        // half-word the next four
        int i1[U][4], i1l[U][4], i2[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          i1[u][0] = i1[u][1] = i1[u][2] = i1[u][3] = 0;
          i1l[u][0] = i1l[u][1] = i1l[u][2] = i1l[u][3] = 0;
          i2[u][0] = i2[u][2] = s2_start[0];
          i2[u][1] = i2[u][3] = s2_start[1];
        }
#pragma unroll
        for (int s = 0; s < Cfg::kSteps8; ++s) {
          const uint4 qc = q_coarse[s * 32];  // q1 b0, q1 b1, q2 b0, q2 b1
          const uint2 qf = q_fine[s * 32];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t xl = iw_lo[u][s], xh = iw_hi[u][s];
            const uint32_t ml = xl & kIdxMask, mh = xh & kIdxMask;
            const uint32_t a[4] = {prmt_ptx(lut_lo[0], lut_lo[1], ml), prmt_ptx(lut_lo[0], lut_lo[1], mh),
                                   prmt_ptx(lut_lo[0], lut_lo[1], ml >> 16),
                                   prmt_ptx(lut_lo[0], lut_lo[1], mh >> 16)};
            mma_s8(i1[u], a, qc.x, qc.y);
            if (ANNA_TQ_FINE_QUERY) mma_s8(i1l[u], a, qf.x, qf.y);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t xl = iw_lo[u][s], xh = iw_hi[u][s];
            const uint32_t a[4] = {prmt_ptx(kTwo, kTwo, xl), prmt_ptx(kTwo, kTwo, xh),
                                   prmt_ptx(kTwo, kTwo, xl >> 16), prmt_ptx(kTwo, kTwo, xh >> 16)};
            mma_s8(i2[u], a, qc.z, qc.w);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            // 254 * coarse + fine stays below 2^31 (|coarse| <= 127 * 127 * D); beta1 carries the 1 / 254
            s1[u][r] = (float)(ANNA_TQ_FINE_QUERY ? i1[u][r] * 254 + i1l[u][r] : i1[u][r]) * beta1[r & 1];
            s2[u][r] = (float)i2[u][r] * beta2[r & 1];
          }
      } else if constexpr (BITS == 2) {
#pragma unroll
        for (int s = 0; s < Cfg::kSteps; ++s) {
          const int h = s % 4;
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t xl = iw_lo[u][s / 4], xh = iw_hi[u][s / 4];
            const uint32_t a[4] = {pm_one_pair(xl, 4 * h, kSignBits, kMinusOne), pm_one_pair(xh, 4 * h, kSignBits, kMinusOne), pm_one_pair(xl, 4 * h + 2, kSignBits, kMinusOne),
                                   pm_one_pair(xh, 4 * h + 2, kSignBits, kMinusOne)};
            mma_f16(s1[u], a, q1f[s][0], q1f[s][1]);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t xl = iw_lo[u][s / 4], xh = iw_hi[u][s / 4];
            const uint32_t a[4] = {pm_one_pair(xl, 4 * h + 1, kSignBits, kMinusOne), pm_one_pair(xh, 4 * h + 1, kSignBits, kMinusOne), pm_one_pair(xl, 4 * h + 3, kSignBits, kMinusOne),
                                   pm_one_pair(xh, 4 * h + 3, kSignBits, kMinusOne)};
            mma_f16(s2[u], a, q2f[s][0], q2f[s][1]);
          }
        }
      } else {
        uint32_t sw_lo[U][Cfg::kSignWords], sw_hi[U][Cfg::kSignWords];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint8_t* signs = st0 + u * Cfg::kStageBytes + Cfg::kOffKey + Cfg::kIdxBytes + tig * (Cfg::kSignWords * 4);
          lds_words<Cfg::kSignWords>(signs + tok_lo * Cfg::kKeyBytes, sw_lo[u]);
          lds_words<Cfg::kSignWords>(signs + tok_hi * Cfg::kKeyBytes, sw_hi[u]);
        }
#pragma unroll
        for (int s = 0; s < Cfg::kSteps; ++s) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            // 2-bit indices: half-word s / 2 of the lane's run, even (s % 2 == 0) or odd fields
            const uint32_t wl = iw_lo[u][s / 4] >> (16 * ((s / 2) % 2) + 2 * (s % 2));
            const uint32_t wh = iw_hi[u][s / 4] >> (16 * ((s / 2) % 2) + 2 * (s % 2));
            const uint32_t sl = wl & 0x3333u, sh = wh & 0x3333u;
            const uint32_t lo_l = prmt(lut_lo[0], lut_lo[1], sl), hi_l = prmt(lut_hi[0], lut_hi[1], sl);
            const uint32_t lo_h = prmt(lut_lo[0], lut_lo[1], sh), hi_h = prmt(lut_hi[0], lut_hi[1], sh);
            const uint32_t a[4] = {prmt(lo_l, hi_l, 0x5140u), prmt(lo_h, hi_h, 0x5140u), prmt(lo_l, hi_l, 0x7362u),
                                   prmt(lo_h, hi_h, 0x7362u)};
            mma_f16(s1[u], a, q1f[s][0], q1f[s][1]);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            // sign plane: bits 2h, 2h + 1 (and + 16) of word s / 8, h = s % 8
            const uint32_t xl = sw_lo[u][s / 8], xh = sw_hi[u][s / 8];
            const int h = s % 8;
            const uint32_t a[4] = {pm_one_pair(xl, 2 * h, kSignBits, kMinusOne), pm_one_pair(xh, 2 * h, kSignBits, kMinusOne), pm_one_pair(xl, 2 * h + 1, kSignBits, kMinusOne),
                                   pm_one_pair(xh, 2 * h + 1, kSignBits, kMinusOne)};
            mma_f16(s2[u], a, q2f[s][0], q2f[s][1]);
          }
        }
      }
    }
    // score (log2 units) = norm * (S1 + rnorm * S2); the constant factors are folded into the query fragments
    float sc[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float* norms = reinterpret_cast<const float*>(st0 + u * Cfg::kStageBytes + Cfg::kOffNorm);
      const float* rnorms = reinterpret_cast<const float*>(st0 + u * Cfg::kStageBytes + Cfg::kOffRnorm);
      const float n_lo = norms[tok_lo], r_lo = rnorms[tok_lo], n_hi = norms[tok_hi], r_hi = rnorms[tok_hi];
      sc[u][0] = n_lo * fmaf(r_lo, s2[u][0], s1[u][0]);
      sc[u][1] = n_lo * fmaf(r_lo, s2[u][1], s1[u][1]);
      sc[u][2] = n_hi * fmaf(r_hi, s2[u][2], s1[u][2]);
      sc[u][3] = n_hi * fmaf(r_hi, s2[u][3], s1[u][3]);
      if (!full) {  // rows past the end of the prefix (their bytes may be anything)
        asm volatile("" ::: "memory");  // a real (warp-uniform) branch: full steps pay nothing for the masking
        if (tok_lo >= valid[u]) sc[u][0] = sc[u][1] = -INFINITY;
        if (tok_hi >= valid[u]) sc[u][2] = sc[u][3] = -INFINITY;
      }
    }

    // ---- online softmax over the U * 16 tokens; the running maximum moves only when it would grow by more than 2^8 ----
    float mx[2] = {fmaxf(sc[0][0], sc[0][2]), fmaxf(sc[0][1], sc[0][3])};
#pragma unroll
    for (int u = 1; u < U; ++u) {
      mx[0] = fmaxf(mx[0], fmaxf(sc[u][0], sc[u][2]));
      mx[1] = fmaxf(mx[1], fmaxf(sc[u][1], sc[u][3]));
    }
#pragma unroll
    for (int d = 4; d <= 16; d <<= 1) {
      mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], d));
      mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], d));
    }
    const bool grew = (mx[0] > m_run[0] + kLazyRescale) || (mx[1] > m_run[1] + kLazyRescale);
    if (__any_sync(0xffffffffu, grew)) {
      const float m_new[2] = {fmaxf(m_run[0], mx[0]), fmaxf(m_run[1], mx[1])};
      const float a0 = fast_exp2(m_run[0] - (m_new[0] == -INFINITY ? 0.0f : m_new[0]));
      const float a1 = fast_exp2(m_run[1] - (m_new[1] == -INFINITY ? 0.0f : m_new[1]));
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
    const float m_ref[2] = {m_run[0] == -INFINITY ? 0.0f : m_run[0], m_run[1] == -INFINITY ? 0.0f : m_run[1]};
    uint32_t pb[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float p0 = fast_exp2(sc[u][0] - m_ref[0]);
      const float p1 = fast_exp2(sc[u][1] - m_ref[1]);
      const float p2 = fast_exp2(sc[u][2] - m_ref[0]);
      const float p3 = fast_exp2(sc[u][3] - m_ref[1]);
      l_run[0] += p0 + p2;
      l_run[1] += p1 + p3;
      pb[u][0] = movmatrix_trans(pack2<__half>(p0, p1));  // rows 2tig, 2tig+1 of head gid
      pb[u][1] = movmatrix_trans(pack2<__half>(p2, p3));  // rows 2tig+8, 2tig+9
    }

    // ---- values: lane holds rows {2tig, 2tig+1} and {2tig+8, 2tig+9}, dims gid*D/8 .. +D/8 -----------------------------------
    uint32_t sc_pair[U][2], zp_pair[U][2];
    uint32_t vw[U][4][Cfg::kValWords];  // rows 2tig, 2tig+1, 2tig+8, 2tig+9
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint8_t* st = st0 + u * Cfg::kStageBytes;
      const T* scales = reinterpret_cast<const T*>(st + Cfg::kOffScale) + v_group;
      const T* zeros = reinterpret_cast<const T*>(st + Cfg::kOffZero) + v_group;
      float sv[4], zv[4];
      const int toks[4] = {tok_a0, tok_a1, tok_a0 + 8, tok_a1 + 8};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sv[i] = ElemTraits<T>::to_float(scales[toks[i] * Cfg::kGroups]);
        zv[i] = ElemTraits<T>::to_float(zeros[toks[i] * Cfg::kGroups]);
      }
      if (!full) {
        asm volatile("" ::: "memory");  // a real (warp-uniform) branch, as above
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (toks[i] >= valid[u]) sv[i] = zv[i] = 0.0f;
      }
      sc_pair[u][0] = pack2<__half>(sv[0], sv[1]);
      sc_pair[u][1] = pack2<__half>(sv[2], sv[3]);
      zp_pair[u][0] = pack2<__half>(zv[0], zv[1]);
      zp_pair[u][1] = pack2<__half>(zv[2], zv[3]);
      const uint8_t* vbase = st + Cfg::kOffVal + gid * (Cfg::kValWords * 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) lds_words<Cfg::kValWords>(vbase + toks[i] * Cfg::kValBytes, vw[u][i]);
    }
    if constexpr (BITS != 2) {
      // 4-bit codes: one 16-bit half-word = 4 dims; x packs the same 4 dims of two tokens (low / high half).  A code
      // moved to bits 6..9 under the exponent of 16 reads as the fp16 number 16 + code, so one fused multiply-add
      // de-quantises a pair: (16 + code) * scale + (zero - 16 * scale).  The shifted zero point is rounded to fp16 once
      // per token and group; it is no larger than the values themselves, so this costs what their own rounding costs.
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) zp_pair[u][pr] = hfma2_u32(sc_pair[u][pr], 0xCC00CC00u, zp_pair[u][pr]);
#pragma unroll
      for (int hw = 0; hw < Cfg::kValWords * 2; ++hw) {
        const uint32_t sel = (hw % 2) ? 0x7632u : 0x5410u;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          uint32_t r[2][4];
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            const uint32_t x = prmt(vw[u][2 * pr][hw / 2], vw[u][2 * pr + 1][hw / 2], sel);
            const uint32_t scl = sc_pair[u][pr], zpt = zp_pair[u][pr];
            r[pr][0] = hfma2_u32(and_or_regs(x << 6, nib_mask, magic16), scl, zpt);
            r[pr][1] = hfma2_u32(and_or_regs(x << 2, nib_mask, magic16), scl, zpt);
            r[pr][2] = hfma2_u32(and_or_regs(x >> 2, nib_mask, magic16), scl, zpt);
            r[pr][3] = hfma2_u32(and_or_regs(x >> 6, nib_mask, magic16), scl, zpt);
          }
          // dims 4hw + {0,1} -> m-tile 2hw (rows gid, gid+8); dims 4hw + {2,3} -> m-tile 2hw + 1
          const uint32_t a_even[4] = {r[0][0], r[0][1], r[1][0], r[1][1]};
          const uint32_t a_odd[4] = {r[0][2], r[0][3], r[1][2], r[1][3]};
          mma_f16(o_acc[2 * hw], a_even, pb[u][0], pb[u][1]);
          mma_f16(o_acc[2 * hw + 1], a_odd, pb[u][0], pb[u][1]);
        }
      }
    } else {
      // 2-bit codes: one 16-bit half-word = 8 dims.  A code moved to bits 8..9 under the exponent of 4 reads as the fp16
      // number 4 + code, so one fused multiply-add de-quantises a pair: (4 + code) * scale + (zero - 4 * scale); the
      // left shifts run on the multiply pipe.
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) zp_pair[u][pr] = hfma2_u32(sc_pair[u][pr], 0xC400C400u, zp_pair[u][pr]);
#pragma unroll
      for (int hw = 0; hw < Cfg::kValWords * 2; ++hw) {
        const uint32_t sel = (hw % 2) ? 0x7632u : 0x5410u;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          uint32_t r[2][8];
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            const uint32_t x = prmt(vw[u][2 * pr][hw / 2], vw[u][2 * pr + 1][hw / 2], sel);
            const uint32_t scl = sc_pair[u][pr], zpt = zp_pair[u][pr];
            r[pr][0] = hfma2_u32(and_or_regs(x << 8, kTwoBitMask, kMagic4), scl, zpt);
            r[pr][1] = hfma2_u32(and_or_regs(x << 6, kTwoBitMask, kMagic4), scl, zpt);
            r[pr][2] = hfma2_u32(and_or_regs(x << 4, kTwoBitMask, kMagic4), scl, zpt);
            r[pr][3] = hfma2_u32(and_or_regs(x << 2, kTwoBitMask, kMagic4), scl, zpt);
            r[pr][4] = hfma2_u32(and_or_regs(x, kTwoBitMask, kMagic4), scl, zpt);
            r[pr][5] = hfma2_u32(and_or_regs(x >> 2, kTwoBitMask, kMagic4), scl, zpt);
            r[pr][6] = hfma2_u32(and_or_regs(x >> 4, kTwoBitMask, kMagic4), scl, zpt);
            r[pr][7] = hfma2_u32(and_or_regs(x >> 6, kTwoBitMask, kMagic4), scl, zpt);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // dims 8hw + {2q, 2q+1} -> m-tile 4hw + q
            const uint32_t a[4] = {r[0][2 * q], r[0][2 * q + 1], r[1][2 * q], r[1][2 * q + 1]};
            mma_f16(o_acc[4 * hw + q], a, pb[u][0], pb[u][1]);
          }
        }
      }
    }
  }
  // ---- merge the four warps; m-tile j holds dims gid*D/8 + 2j (row gid) and + 2j + 1 (row gid + 8) --------------------------
#pragma unroll
  for (int d = 4; d <= 16; d <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], d);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], d);
  }
  __syncthreads();
  float* sm_m = reinterpret_cast<float*>(smem_raw);
  float* sm_l = sm_m + kMmaWarps * 8;
  float* sm_o = sm_l + kMmaWarps * 8;
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
    const int dim = gid * (D / 8) + 2 * j;
    base[(2 * tig) * kPad + dim] = o_acc[j][0];
    base[(2 * tig + 1) * kPad + dim] = o_acc[j][1];
    base[(2 * tig) * kPad + dim + 1] = o_acc[j][2];
    base[(2 * tig + 1) * kPad + dim + 1] = o_acc[j][3];
  }
  __syncthreads();
  const int64_t part = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity + out_slot;
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
      stats_out[(int64_t)g * p.chunk_capacity * 2 + 0] = m_all * 0.6931471805599453f;
      stats_out[(int64_t)g * p.chunk_capacity * 2 + 1] = l_all;
    }
  }
  // The window kernel's partials and, when it arrives last, its merged output must be complete before this CTA
  // counts itself in (fused merge) or the kernel ends (two-pass merge).
  wait_for_prior_grids();
  if (p.fused.counters != nullptr) {
    const int64_t head0 = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity;
    __syncthreads();
    fused_combine_tail<T, D, kMmaThreads>(p.fused, b, hq0, g_count, active_chunks, p.chunk_capacity,
                                          p.stats + head0 * 2, p.values + head0 * D,
                                          reinterpret_cast<float*>(smem_raw), (int64_t)b * gridDim.y + blockIdx.y);
  }
}

template <typename T, int D, int BITS>
static int launch_tq_mma(const TqDecodeParams& p, int batch, cudaStream_t stream) {
  using Cfg = TqMmaCfg<T, D, BITS>;
  auto kernel = tq_decode_split_mma_kernel<T, D, BITS>;
  static bool configured[64] = {};
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !configured[device]) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(tq_window_split_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         MmaCfg<D>::kSmemBytes));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  // with 16-token pages a tile is copied as one run, so the page chunk must have exactly the stage's layout
  if (p.block_size == kTileTokens &&
      (p.layout.off_kcodes != Cfg::kOffKey || p.layout.off_knorm != Cfg::kOffNorm ||
       p.layout.off_krnorm != Cfg::kOffRnorm || p.layout.off_vdata != Cfg::kOffVal ||
       p.layout.off_vscale != Cfg::kOffScale || p.layout.off_vzero != Cfg::kOffZero ||
       p.layout.chunk_bytes < Cfg::kTileDataBytes))
    return set_error(ANNA_ERR_INVALID, "packed page layout does not match the decode kernel's tile layout");
  const int group_tiles = (p.groups + 7) / 8;
  dim3 prep_grid((unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
  tq_prepare_queries_kernel<T, D, BITS><<<prep_grid, kMmaThreads, 0, stream>>>(p);
  int rc = check_launch("tq_prepare_queries_kernel");
  if (rc != ANNA_OK) return rc;
  dim3 window_grid((unsigned)p.num_window_chunks, (unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
  tq_window_split_mma_kernel<T, D><<<window_grid, kMmaThreads, MmaCfg<D>::kSmemBytes, stream>>>(p);
  rc = check_launch("tq_window_split_mma_kernel");
  if (rc != ANNA_OK) return rc;
  if (p.num_chunks > p.num_window_chunks) {
    dim3 grid((unsigned)p.num_chunks, (unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
#if ANNA_TQ_OVERLAP_WINDOW
    // programmatic dependent launch: the packed chunks run beside the (small) window launch instead of after it; the
    // query fragments they read come from the launch before that one, which has completed by then
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(kMmaThreads);
    config.dynamicSmemBytes = Cfg::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    ANNA_CUDA_CHECK(cudaLaunchKernelEx(&config, kernel, p));
#else
    kernel<<<grid, kMmaThreads, Cfg::kSmemBytes, stream>>>(p);
#endif
    rc = check_launch("tq_decode_split_mma_kernel");
  }
  return rc;
}

template <typename T, int D>
static int launch_window(const TqDecodeParams& p, int batch, cudaStream_t stream) {
  static bool configured[64] = {};
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !configured[device]) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(tq_window_split_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         MmaCfg<D>::kSmemBytes));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  const int group_tiles = (p.groups + 7) / 8;
  dim3 window_grid((unsigned)p.num_window_chunks, (unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
  tq_window_split_mma_kernel<T, D><<<window_grid, kMmaThreads, MmaCfg<D>::kSmemBytes, stream>>>(p);
  return check_launch("tq_window_split_mma_kernel");
}

int launch_tq_window_split(const TqDecodeParams& p, int batch, int head_dim, int dtype, cudaStream_t stream) {
  if (dtype == ANNA_DTYPE_BF16)
    return head_dim == 128 ? launch_window<__nv_bfloat16, 128>(p, batch, stream)
                           : launch_window<__nv_bfloat16, 256>(p, batch, stream);
  return head_dim == 128 ? launch_window<__half, 128>(p, batch, stream) : launch_window<__half, 256>(p, batch, stream);
}

int tq_decode_mma_faults(int* count) {
  int32_t value = 0;
  ANNA_CUDA_CHECK(cudaMemcpyFromSymbol(&value, g_tq_mma_faults, sizeof(value)));
  *count = (int)value;
  return ANNA_OK;
}

// Self-test of the bounded wait: nobody ever arrives on this barrier, so the wait has to give up and say so.
__global__ void wait_expiry_selftest_kernel(int32_t* result) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  __syncwarp();
  const bool landed = mbar_wait(bar, 0u);
  if (threadIdx.x == 0) *result = landed ? 0 : 1;
}

bool tq_split_mma_applicable(const TqDecodeParams& p, int head_dim, int dtype) {
  static const bool disabled = [] {
    const char* flag = std::getenv("ANNA_B200_DISABLE_MMA");
    return flag != nullptr && flag[0] != '\0' && flag[0] != '0';
  }();
  if (disabled) return false;
  if (dtype != ANNA_DTYPE_F16 && dtype != ANNA_DTYPE_BF16) return false;
  if (head_dim != 128 && head_dim != 256) return false;
  if (p.value_group != 32 || p.block_size % kTileTokens != 0 || p.chunk_tokens % kTileTokens != 0) return false;
  if (p.max_len >= (int64_t)1 << 31 || p.query_frags == nullptr) return false;
  return true;
}

int launch_tq_split_mma(const TqDecodeParams& p, int batch, int head_dim, int bits, int dtype, cudaStream_t stream) {
#define ANNA_TQ_MMA_CASE(TYPE, DIM, BITS_) \
  if (head_dim == DIM && bits == BITS_) return launch_tq_mma<TYPE, DIM, BITS_>(p, batch, stream);
  if (dtype == ANNA_DTYPE_BF16) {
    ANNA_TQ_MMA_CASE(__nv_bfloat16, 128, 2) ANNA_TQ_MMA_CASE(__nv_bfloat16, 128, 3) ANNA_TQ_MMA_CASE(__nv_bfloat16, 128, 4)
    ANNA_TQ_MMA_CASE(__nv_bfloat16, 256, 2) ANNA_TQ_MMA_CASE(__nv_bfloat16, 256, 3) ANNA_TQ_MMA_CASE(__nv_bfloat16, 256, 4)
  } else {
    ANNA_TQ_MMA_CASE(__half, 128, 2) ANNA_TQ_MMA_CASE(__half, 128, 3) ANNA_TQ_MMA_CASE(__half, 128, 4)
    ANNA_TQ_MMA_CASE(__half, 256, 2) ANNA_TQ_MMA_CASE(__half, 256, 3) ANNA_TQ_MMA_CASE(__half, 256, 4)
  }
#undef ANNA_TQ_MMA_CASE
  return set_error(ANNA_ERR_UNSUPPORTED, "no tensor-core TurboQuant decode for head_dim %d, %d bits", head_dim, bits);
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
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(&value, flag, sizeof(value), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize((cudaStream_t)stream);
  cudaFree(flag);
  if (err != cudaSuccess)
    return anna::set_error(ANNA_ERR_CUDA, "wait-expiry self-test failed: %s", cudaGetErrorString(err));
  *expired = (int)value;
  return ANNA_OK;
}

// Number of bounded waits that expired in the kernels that stage tiles with the copy engine, on the current device,
// since the library was loaded (0 in a healthy run).  Synchronises the device.
extern "C" int anna_kv_device_faults(int* count) {
  ANNA_REQUIRE(count != nullptr, "anna_kv_device_faults: null output pointer");
  int mma = 0, umma = 0, prefill = 0;
  int rc = anna::tq_decode_mma_faults(&mma);
  if (rc == ANNA_OK) rc = anna::tq_decode_umma_faults(&umma);
  if (rc == ANNA_OK) rc = anna::prefill_umma_faults(&prefill);
  if (rc != ANNA_OK) return rc;
  *count = mma + umma + prefill;
  return ANNA_OK;
}
