// MSE-only TurboQuant codes for a plain tensor row (the K or V history of one sequence in Anna's Gemma4 runtime):
// every [head_dim] vector becomes b-bit Lloyd-Max indices of its normalised, rotated coordinates plus its norm.
//   quantize:   x -> ||x||, w = fwht(s1 * x) / ||x||, idx_d = #{boundaries < w_d}
//   dequantize: a_d = centroid[idx_d], x_hat = (||x|| / D) * s1 * fwht(a)
// One warp per vector, coordinates e0 .. e0 + D/32 per lane; the arithmetic order (pairwise tree sums, butterfly order,
// correctly rounded fp32 operations) is the one of the CPU restatement, so the indices match it bit for bit.
// Packed row of a vector: b = 2 -> 4 indices per byte, b = 3 / 4 -> 2 per byte (4-bit fields), low field first.
#include "tq_common.cuh"

namespace anna {

constexpr int kTensorWarps = 8;

struct TqTensorParams {
  const void* x;            // quantize: source vectors; dequantize: unused
  void* out;                // dequantize: destination vectors
  int64_t stride_h, stride_t;   // element strides of x / out: head, token (last dim contiguous)
  uint8_t* idx;             // [heads, capacity, row_bytes]
  float* norms;             // [heads, capacity]
  int64_t capacity;         // tokens per head the code buffers can hold
  int64_t offset;           // first token position inside the code buffers
  int heads, tokens;
  const float* signs1;
  const float* centroids;
  const float* boundaries;
};

template <int D, int BITS>
struct TensorCodeLayout {
  static constexpr int kFieldBits = BITS == 2 ? 2 : 4;
  static constexpr int kRowBytes = D * kFieldBits / 8;
};

template <typename T, int D, int BITS>
__global__ void __launch_bounds__(kTensorWarps * 32) tq_tensor_quantize_kernel(const TqTensorParams p) {
  constexpr int E = D / 32;
  constexpr int NB = (1 << BITS) - 1;
  using Layout = TensorCodeLayout<D, BITS>;
  const int lane = threadIdx.x & 31;
  const int e0 = lane * E;
  uint32_t flips = 0;
#pragma unroll
  for (int j = 0; j < E; ++j) flips |= (p.signs1[e0 + j] < 0.0f ? 1u : 0u) << j;
  float bnd[NB];
#pragma unroll
  for (int k = 0; k < NB; ++k) bnd[k] = p.boundaries[k];
  const int64_t total = (int64_t)p.heads * p.tokens;
  const int64_t warps = (int64_t)gridDim.x * kTensorWarps;
  for (int64_t item = (int64_t)blockIdx.x * kTensorWarps + (threadIdx.x >> 5); item < total; item += warps) {
    const int h = (int)(item / p.tokens);
    const int t = (int)(item - (int64_t)h * p.tokens);
    float x[E], w[E], sq[E];
    lane_load<T, E>(reinterpret_cast<const T*>(p.x) + (int64_t)h * p.stride_h + (int64_t)t * p.stride_t + e0, x);
#pragma unroll
    for (int j = 0; j < E; ++j) sq[j] = __fmul_rn(x[j], x[j]);
    const float norm = __fsqrt_rn(warp_tree_sum<E>(sq));
    const float inv = __frcp_rn(fmaxf(norm, 1e-20f));
#pragma unroll
    for (int j = 0; j < E; ++j) w[j] = __uint_as_float(__float_as_uint(x[j]) ^ ((flips >> j) << 31));
    warp_fwht<E>(w, lane);
    uint64_t field = 0;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float scaled = __fmul_rn(w[j], inv);
      uint32_t c = 0;
#pragma unroll
      for (int k = 0; k < NB; ++k) c += scaled > bnd[k] ? 1u : 0u;
      field |= (uint64_t)c << (Layout::kFieldBits * j);
    }
    const int64_t slot = (int64_t)h * p.capacity + p.offset + t;
    warp_pack_store<Layout::kFieldBits * E>(field, p.idx + slot * Layout::kRowBytes, lane);
    if (lane == 0) p.norms[slot] = norm;
  }
}

template <typename T, int D, int BITS>
__global__ void __launch_bounds__(kTensorWarps * 32) tq_tensor_dequantize_kernel(const TqTensorParams p) {
  constexpr int E = D / 32;
  using Layout = TensorCodeLayout<D, BITS>;
  constexpr int kFieldBits = Layout::kFieldBits;
  constexpr int kLaneBits = kFieldBits * E;  // 4 .. 64 bits of the packed row belong to one lane
  __shared__ float sm_cent[1 << BITS];
  if (threadIdx.x < (1 << BITS)) sm_cent[threadIdx.x] = p.centroids[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int e0 = lane * E;
  uint32_t flips = 0;
#pragma unroll
  for (int j = 0; j < E; ++j) flips |= (p.signs1[e0 + j] < 0.0f ? 1u : 0u) << j;
  constexpr float inv_dim = 1.0f / (float)D;
  const int64_t total = (int64_t)p.heads * p.tokens;
  const int64_t warps = (int64_t)gridDim.x * kTensorWarps;
  for (int64_t item = (int64_t)blockIdx.x * kTensorWarps + (threadIdx.x >> 5); item < total; item += warps) {
    const int h = (int)(item / p.tokens);
    const int t = (int)(item - (int64_t)h * p.tokens);
    const int64_t slot = (int64_t)h * p.capacity + p.offset + t;
    const uint8_t* row = p.idx + slot * Layout::kRowBytes;
    uint64_t field;
    if constexpr (kLaneBits == 64) {
      const uint2 v = reinterpret_cast<const uint2*>(row)[lane];
      field = (uint64_t)v.x | ((uint64_t)v.y << 32);
    } else if constexpr (kLaneBits == 32) {
      field = reinterpret_cast<const uint32_t*>(row)[lane];
    } else {
      constexpr int kLanesPerWord = 32 / kLaneBits;
      const uint32_t word = reinterpret_cast<const uint32_t*>(row)[lane / kLanesPerWord];
      field = (word >> ((lane % kLanesPerWord) * kLaneBits)) & ((1u << kLaneBits) - 1u);
    }
    float a[E];
#pragma unroll
    for (int j = 0; j < E; ++j) a[j] = sm_cent[(uint32_t)(field >> (kFieldBits * j)) & ((1u << kFieldBits) - 1u)];
    warp_fwht<E>(a, lane);
    const float scale = __fmul_rn(p.norms[slot], inv_dim);
    T* dst = reinterpret_cast<T*>(p.out) + (int64_t)h * p.stride_h + (int64_t)t * p.stride_t + e0;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float signed_a = __uint_as_float(__float_as_uint(a[j]) ^ ((flips >> j) << 31));
      dst[j] = ElemTraits<T>::from_float(__fmul_rn(scale, signed_a));
    }
  }
}

#define ANNA_DISPATCH_TENSOR_DIM(dim, D, ...)                                                                          \
  [&]() -> int {                                                                                                       \
    switch (dim) {                                                                                                     \
      case 64: { constexpr int D = 64; return __VA_ARGS__(); }                                                         \
      case 128: { constexpr int D = 128; return __VA_ARGS__(); }                                                       \
      case 256: { constexpr int D = 256; return __VA_ARGS__(); }                                                       \
      case 512: { constexpr int D = 512; return __VA_ARGS__(); }                                                       \
      default: return ::anna::set_error(ANNA_ERR_UNSUPPORTED, "unsupported head_dim %d (64, 128, 256, 512)", (int)(dim)); \
    }                                                                                                                  \
  }()

static int check_tensor_args(const char* what, int heads, int tokens, int head_dim, int bits, int dtype,
                             int64_t stride_h, int64_t stride_t, int64_t capacity, int64_t offset) {
  if (heads <= 0 || tokens <= 0) return set_error(ANNA_ERR_INVALID, "%s: heads and tokens must be positive", what);
  if (offset < 0 || offset + tokens > capacity)
    return set_error(ANNA_ERR_WORKSPACE, "%s: tokens [%lld, %lld) do not fit code buffers of %lld tokens", what,
                     (long long)offset, (long long)(offset + tokens), (long long)capacity);
  const int vec = dtype == ANNA_DTYPE_F32 ? 4 : 8;
  const int lane_elems = head_dim / 32;
  // a lane reads / writes head_dim / 32 contiguous elements with one aligned access
  const int align = lane_elems < vec ? lane_elems : vec;
  if (stride_h % align != 0 || stride_t % align != 0)
    return set_error(ANNA_ERR_INVALID, "%s: strides must keep every lane's elements aligned", what);
  (void)bits;
  return ANNA_OK;
}

}  // namespace anna

using namespace anna;

extern "C" int anna_tq_tensor_row_bytes(int head_dim, int bits) {
  if (head_dim <= 0 || head_dim % 32 != 0 || bits < 2 || bits > 4) return -1;
  return head_dim * (bits == 2 ? 2 : 4) / 8;
}

extern "C" int anna_tq_tensor_quantize(const void* x, int64_t stride_h, int64_t stride_t, uint8_t* idx, float* norms,
                                       int64_t capacity, int64_t offset, int heads, int tokens, int head_dim, int bits,
                                       const float* signs1, const float* boundaries, int dtype, anna_stream_t stream) {
  ANNA_REQUIRE(x && idx && norms && signs1 && boundaries, "anna_tq_tensor_quantize: null pointer argument");
  int rc = check_tensor_args("anna_tq_tensor_quantize", heads, tokens, head_dim, bits, dtype, stride_h, stride_t, capacity,
                             offset);
  if (rc != ANNA_OK) return rc;
  TqTensorParams p{};
  p.x = x; p.stride_h = stride_h; p.stride_t = stride_t; p.idx = idx; p.norms = norms; p.capacity = capacity;
  p.offset = offset; p.heads = heads; p.tokens = tokens; p.signs1 = signs1; p.boundaries = boundaries;
  const int64_t total = (int64_t)heads * tokens;
  int64_t blocks = (total + kTensorWarps - 1) / kTensorWarps;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    return ANNA_DISPATCH_TENSOR_DIM(head_dim, D, [&]() -> int {
      return ANNA_DISPATCH_TQ_BITS(bits, BITS, [&]() -> int {
        tq_tensor_quantize_kernel<T, D, BITS><<<(unsigned)blocks, kTensorWarps * 32, 0, (cudaStream_t)stream>>>(p);
        return check_launch("tq_tensor_quantize_kernel");
      });
    });
  });
}

extern "C" int anna_tq_tensor_dequantize(const uint8_t* idx, const float* norms, int64_t capacity, int64_t offset,
                                         void* out, int64_t stride_h, int64_t stride_t, int heads, int tokens,
                                         int head_dim, int bits, const float* signs1, const float* centroids, int dtype,
                                         anna_stream_t stream) {
  ANNA_REQUIRE(idx && norms && out && signs1 && centroids, "anna_tq_tensor_dequantize: null pointer argument");
  int rc = check_tensor_args("anna_tq_tensor_dequantize", heads, tokens, head_dim, bits, dtype, stride_h, stride_t,
                             capacity, offset);
  if (rc != ANNA_OK) return rc;
  TqTensorParams p{};
  p.out = out; p.stride_h = stride_h; p.stride_t = stride_t; p.idx = const_cast<uint8_t*>(idx);
  p.norms = const_cast<float*>(norms); p.capacity = capacity; p.offset = offset; p.heads = heads; p.tokens = tokens;
  p.signs1 = signs1; p.centroids = centroids;
  const int64_t total = (int64_t)heads * tokens;
  int64_t blocks = (total + kTensorWarps - 1) / kTensorWarps;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    return ANNA_DISPATCH_TENSOR_DIM(head_dim, D, [&]() -> int {
      return ANNA_DISPATCH_TQ_BITS(bits, BITS, [&]() -> int {
        tq_tensor_dequantize_kernel<T, D, BITS><<<(unsigned)blocks, kTensorWarps * 32, 0, (cudaStream_t)stream>>>(p);
        return check_launch("tq_tensor_dequantize_kernel");
      });
    });
  });
}
