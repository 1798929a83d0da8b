// TurboQuant building blocks shared by the append, decode and materialize kernels.
//
// Vector-per-warp convention: a head_dim-D vector lives in one warp, lane l holding the E = D / 32 contiguous
// coordinates [l*E, (l+1)*E).  The Walsh-Hadamard butterflies and the pairwise tree sums below visit pairs in the
// order "stride 1, 2, 4, ... D/2", adjacent pairs first, with every add / sub / mul issued through the _rn
// intrinsics, so the results are bitwise those of a scalar loop that walks the same network.
#pragma once

#include "common.cuh"

namespace anna {

__host__ __device__ inline int align_up(int v, int to) { return (v + to - 1) / to * to; }

// Fills the layout of one (page, kv head) chunk; returns false for unsupported geometry.
__host__ __device__ inline bool tq_make_layout(int head_dim, int bits, int block_size, int dtype_bytes, int group,
                                               anna_tq_layout* out) {
  if (bits < 2 || bits > 4 || head_dim <= 0 || block_size <= 0 || group <= 0 || head_dim % group != 0) return false;
  if ((head_dim * bits) % 8 != 0) return false;
  out->key_bytes = head_dim * bits / 8;
  out->value_bytes = head_dim / (bits == 2 ? 4 : 2);
  out->groups = head_dim / group;
  out->off_kcodes = 0;
  out->off_knorm = align_up(block_size * out->key_bytes, 16);
  out->off_krnorm = align_up(out->off_knorm + 4 * block_size, 16);
  out->off_vdata = align_up(out->off_krnorm + 4 * block_size, 16);
  out->off_vscale = align_up(out->off_vdata + block_size * out->value_bytes, 16);
  out->off_vzero = align_up(out->off_vscale + block_size * out->groups * dtype_bytes, 16);
  out->chunk_bytes = align_up(out->off_vzero + block_size * out->groups * dtype_bytes, 128);
  return true;
}

inline int dtype_bytes_of(int dtype) { return dtype == ANNA_DTYPE_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------------------------------------------
// warp-resident vector primitives

template <int E>
__device__ __forceinline__ void warp_fwht(float (&w)[E], int lane) {
#pragma unroll
  for (int h = 1; h < E; h <<= 1) {
#pragma unroll
    for (int j = 0; j < E; ++j) {
      if ((j & h) == 0) {
        const float lo = w[j], hi = w[j + h];
        w[j] = __fadd_rn(lo, hi);
        w[j + h] = __fsub_rn(lo, hi);
      }
    }
  }
#pragma unroll
  for (int dl = 1; dl < 32; dl <<= 1) {
    // lower lane: w + other, upper lane: other - w.  One fused multiply-add by +-1 rounds exactly like the add / sub.
    const float sgn = (lane & dl) != 0 ? -1.0f : 1.0f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, w[j], dl);
      w[j] = __fmaf_rn(w[j], sgn, other);
    }
  }
}

// Pairwise tree sum of E per-lane values over the whole warp; every lane gets the total.
template <int E>
__device__ __forceinline__ float warp_tree_sum(float (&t)[E]) {
#pragma unroll
  for (int h = 1; h < E; h <<= 1) {
#pragma unroll
    for (int j = 0; j < E; j += 2 * h) t[j] = __fadd_rn(t[j], t[j + h]);
  }
  float s = t[0];
#pragma unroll
  for (int dl = 1; dl < 32; dl <<= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, dl));
  return s;
}

// Store one packed row: lane l contributes the W-bit field `field` for bit positions [l*W, (l+1)*W).
// dst must be 4-byte aligned.  With `enabled` false (warp-uniform) the warp takes part in the exchange but stores nothing.
template <int W>
__device__ __forceinline__ void warp_pack_store(uint64_t field, uint8_t* __restrict__ dst, int lane, bool enabled = true) {
  if constexpr (W == 64) {
    uint32_t* out = reinterpret_cast<uint32_t*>(dst) + lane * 2;
    if (enabled) {
      out[0] = (uint32_t)field;
      out[1] = (uint32_t)(field >> 32);
    }
  } else if constexpr (W == 32) {
    if (enabled) reinterpret_cast<uint32_t*>(dst)[lane] = (uint32_t)field;
  } else {
    constexpr int kLanesPerWord = 32 / W;
    uint32_t word = (uint32_t)field << ((lane % kLanesPerWord) * W);
#pragma unroll
    for (int dl = 1; dl < kLanesPerWord; dl <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, dl);
    if (enabled && lane % kLanesPerWord == 0) reinterpret_cast<uint32_t*>(dst)[lane / kLanesPerWord] = word;
  }
}

// Lane-local contiguous load / store of E elements (E * sizeof(T) is 4, 8, 16 or a multiple of 16 bytes).
template <typename T, int E>
__device__ __forceinline__ void lane_load(const T* __restrict__ ptr, float (&dst)[E]) {
  constexpr int kBytes = E * (int)sizeof(T);
  if constexpr (kBytes % 16 == 0) {
    constexpr int kVec = ElemTraits<T>::kVec;
#pragma unroll
    for (int c = 0; c < kBytes / 16; ++c) {
      float piece[kVec];
      widen16<T>(*reinterpret_cast<const uint4*>(ptr + c * kVec), piece);
#pragma unroll
      for (int i = 0; i < kVec; ++i) dst[c * kVec + i] = piece[i];
    }
  } else {
    T tmp[E];
    if constexpr (kBytes == 8) {
      *reinterpret_cast<uint2*>(tmp) = *reinterpret_cast<const uint2*>(ptr);
    } else {
      static_assert(kBytes == 4, "unsupported lane width");
      *reinterpret_cast<uint32_t*>(tmp) = *reinterpret_cast<const uint32_t*>(ptr);
    }
#pragma unroll
    for (int i = 0; i < E; ++i) dst[i] = ElemTraits<T>::to_float(tmp[i]);
  }
}

template <typename T, int E>
__device__ __forceinline__ void lane_copy(const T* __restrict__ src, T* __restrict__ dst) {
  constexpr int kBytes = E * (int)sizeof(T);
  if constexpr (kBytes % 16 == 0) {
#pragma unroll
    for (int c = 0; c < kBytes / 16; ++c)
      reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
  } else if constexpr (kBytes == 8) {
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
  } else {
    static_assert(kBytes == 4, "unsupported lane width");
    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
  }
}

// (float)(1 / sqrt(D)), correctly rounded, for the supported power-of-two head dims.
template <int D>
__host__ __device__ constexpr float rsqrt_dim_const() {
  static_assert(D == 32 || D == 64 || D == 128 || D == 256 || D == 512, "unsupported head_dim");
  return D == 32 ? 0.17677669529663687f
       : D == 64 ? 0.125f
       : D == 128 ? 0.08838834764831845f
       : D == 256 ? 0.0625f
                  : 0.044194173824159216f;
}

template <typename T>
__device__ __forceinline__ float round_to_elem(float v) {
  return ElemTraits<T>::to_float(ElemTraits<T>::from_float(v));
}

#define ANNA_DISPATCH_TQ_DIM(dim, D, ...)                                                    \
  [&]() -> int {                                                                             \
    switch (dim) {                                                                           \
      case 64: { constexpr int D = 64; return __VA_ARGS__(); }                               \
      case 128: { constexpr int D = 128; return __VA_ARGS__(); }                             \
      case 256: { constexpr int D = 256; return __VA_ARGS__(); }                             \
      default: return ::anna::set_error(ANNA_ERR_UNSUPPORTED, "unsupported TurboQuant head_dim %d (64, 128, 256)", (int)(dim)); \
    }                                                                                        \
  }()

#define ANNA_DISPATCH_TQ_BITS(bits, BITS, ...)                                               \
  [&]() -> int {                                                                             \
    switch (bits) {                                                                          \
      case 2: { constexpr int BITS = 2; return __VA_ARGS__(); }                              \
      case 3: { constexpr int BITS = 3; return __VA_ARGS__(); }                              \
      case 4: { constexpr int BITS = 4; return __VA_ARGS__(); }                              \
      default: return ::anna::set_error(ANNA_ERR_UNSUPPORTED, "unsupported TurboQuant bit-width %d (2, 3, 4)", (int)(bits)); \
    }                                                                                        \
  }()

}  // namespace anna
