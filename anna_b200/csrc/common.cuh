// Shared device/host helpers for libanna_b200_kv (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/anna_b200_kv.h"

namespace anna {

// ---------------------------------------------------------------------------------------------------------------
// host-side status plumbing

int set_error(int code, const char* fmt, ...);  // formats into the thread-local message, returns `code`

#define ANNA_REQUIRE(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::anna::set_error(ANNA_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define ANNA_CUDA_CHECK(expr)                                                                        \
  do {                                                                                               \
    cudaError_t err__ = (expr);                                                                      \
    if (err__ != cudaSuccess)                                                                        \
      return ::anna::set_error(ANNA_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));    \
  } while (0)

constexpr int kMaxPeerOutputs = 7;  // the other GPUs of an 8-GPU box

inline int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return set_error(ANNA_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(err));
  return ANNA_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// element types

template <typename T>
struct ElemTraits;

template <>
struct ElemTraits<float> {
  static constexpr int kVec = 4;  // elements per 16-byte load
  static __device__ __forceinline__ float to_float(float v) { return v; }
  static __device__ __forceinline__ float from_float(float v) { return v; }
};
template <>
struct ElemTraits<__half> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <>
struct ElemTraits<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// Load kVec contiguous elements (16 bytes, 16-byte aligned) and widen to float.
template <typename T>
__device__ __forceinline__ void load_vec16(const T* __restrict__ ptr, float (&dst)[ElemTraits<T>::kVec]);

template <>
__device__ __forceinline__ void load_vec16<float>(const float* __restrict__ ptr, float (&dst)[4]) {
  const float4 v = __ldg(reinterpret_cast<const float4*>(ptr));
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
template <>
__device__ __forceinline__ void load_vec16<__half>(const __half* __restrict__ ptr, float (&dst)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(ptr));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    const float2 f = __half22float2(h);
    dst[2 * i] = f.x;
    dst[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load_vec16<__nv_bfloat16>(const __nv_bfloat16* __restrict__ ptr, float (&dst)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(ptr));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dst[2 * i] = __uint_as_float(w[i] << 16);
    dst[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// Streaming variant: bypass L1 allocation for data that is read once.
template <typename T>
__device__ __forceinline__ uint4 ldg_stream16(const T* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

template <typename T>
__device__ __forceinline__ void widen16(const uint4& v, float (&dst)[ElemTraits<T>::kVec]);
template <>
__device__ __forceinline__ void widen16<float>(const uint4& v, float (&dst)[4]) {
  dst[0] = __uint_as_float(v.x); dst[1] = __uint_as_float(v.y);
  dst[2] = __uint_as_float(v.z); dst[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void widen16<__half>(const uint4& v, float (&dst)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    dst[2 * i] = f.x;
    dst[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void widen16<__nv_bfloat16>(const uint4& v, float (&dst)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dst[2 * i] = __uint_as_float(w[i] << 16);
    dst[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

#define ANNA_DISPATCH_DTYPE(dtype, T, ...)                                                   \
  [&]() -> int {                                                                             \
    switch (dtype) {                                                                         \
      case ANNA_DTYPE_F32: { using T = float; return __VA_ARGS__(); }                        \
      case ANNA_DTYPE_F16: { using T = __half; return __VA_ARGS__(); }                       \
      case ANNA_DTYPE_BF16: { using T = __nv_bfloat16; return __VA_ARGS__(); }               \
      default: return ::anna::set_error(ANNA_ERR_UNSUPPORTED, "unsupported dtype code %d", (int)(dtype)); \
    }                                                                                        \
  }()

__device__ __forceinline__ float sigmoidf_fast(float x) { return 1.0f / (1.0f + __expf(-x)); }

// ---------------------------------------------------------------------------------------------------------------
// split-K partials, owned by the caller:
//   stats  float [B, Hq, chunk_capacity, 2]  (running max, denominator)
//   values float [B, Hq, chunk_capacity, D]
struct SplitWorkspace {
  float* stats;
  float* values;
  int chunk_capacity;  // stride (in chunks) between consecutive query heads
};

// Resolves the chunking of a decode call: chunk_tokens == 0 asks for the automatic plan, otherwise the caller's
// chunk length is used as is (the reference's split-K block size).  Fails when the partial buffers are too small.
int resolve_split(int batch, int kv_heads, int64_t max_len, int chunk_tokens_in, int chunk_capacity,
                  const float* partial_stats, const float* partial_values, int* chunk_tokens, int* num_chunks);

// Launches the combine pass (defined in combine.cu).  lengths32 / lengths64: at most one is non-null; with both
// null every row has fixed_len keys.  max_len clamps like the split pass.  window > 0 selects the TurboQuant slot
// count (window chunks + packed chunks).
int launch_split_combine(const SplitWorkspace& ws, const int32_t* lengths32, const int64_t* lengths64,
                         int64_t fixed_len, int64_t max_len, int window, const void* gate, int64_t gate_stride_b,
                         int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h, int batch,
                         int q_heads, int head_dim, int chunk_tokens, int num_chunks, int dtype, cudaStream_t stream);

}  // namespace anna
