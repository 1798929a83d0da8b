// De-quantize packed TurboQuant pages into dense keys / values in the cache dtype (a warp per run of token-heads); with the
// window ring given, the same launch also copies the un-quantized tail of every row and zero-pads up to max_len, i.e.
// it produces the whole dense view of a batch of rows.
#include "tq_common.cuh"

namespace anna {

struct TqMaterializeParams {
  const uint8_t* pages;
  const int32_t* block_table;
  int64_t table_stride;
  const int64_t* quantized_lengths;
  const float* signs1;
  const float* signs2;
  const float* centroids;
  void* key_out;
  void* value_out;
  int64_t out_stride_b, out_stride_h, out_stride_t;
  int kv_heads, block_size, value_group;
  int64_t num_pages, max_blocks, max_quantized_len;
  anna_tq_layout layout;
  // optional dense tail: window ring [slots, 2, Hkv, R, D], ring slot and total length per row
  const void* window;
  const int64_t* window_slots;
  const int64_t* lengths;
  int residual_len;
};

constexpr int kMaterializeWarps = 4;
constexpr int kMaterializeTokens = 8;  // consecutive tokens of one (row, kv head) per warp

// A warp walks kMaterializeTokens consecutive tokens of one (row, kv head): the sign vectors stay in registers, the
// codes of a token are one 2- or 4-byte load per lane where the geometry allows, and two tokens are in flight at a time
// so that the shuffles of one transform hide behind the arithmetic of the other.  The arithmetic per token is unchanged
// (same order of operations as the one-token-per-warp version it replaces), so the output is bit-identical.
template <typename T, int D, int BITS>
__global__ void __launch_bounds__(kMaterializeWarps * 32) tq_materialize_kernel(const TqMaterializeParams p) {
  constexpr int E = D / 32;
  constexpr int M = BITS - 1;
  constexpr int VS = BITS == 2 ? 2 : 4;
  __shared__ float sm_cent[1 << M];
  if (threadIdx.x < (1 << M)) sm_cent[threadIdx.x] = p.centroids[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int e0 = lane * E;
  const int64_t t0 = ((int64_t)blockIdx.x * kMaterializeWarps + warp) * kMaterializeTokens;
  if (t0 >= p.max_quantized_len) return;

  const bool dense_view = p.window != nullptr;
  int64_t len = 0, lq;
  if (dense_view) {
    // whole dense view: [0, len - R) from the pages, [len - R, len) from the ring, [len, max) zeros
    // (max_quantized_len is the padded length in this mode)
    len = max((int64_t)0, min(p.lengths[b], p.max_quantized_len));
    lq = len > p.residual_len ? len - p.residual_len : 0;
  } else {
    lq = min(p.quantized_lengths[b], p.max_quantized_len);
  }
  float s1[E], s2[E];
#pragma unroll
  for (int j = 0; j < E; ++j) {
    s1[j] = p.signs1[e0 + j];
    s2[j] = p.signs2[e0 + j];
  }
  const int64_t out_base = (int64_t)b * p.out_stride_b + (int64_t)h * p.out_stride_h + e0;
  const int64_t t_end = min(t0 + kMaterializeTokens, p.max_quantized_len);

#pragma unroll 2
  for (int64_t t = t0; t < t_end; ++t) {
    T* kout = reinterpret_cast<T*>(p.key_out) + out_base + t * p.out_stride_t;
    T* vout = reinterpret_cast<T*>(p.value_out) + out_base + t * p.out_stride_t;
    if (t >= lq) {
      if (!dense_view) break;
      if (t < len) {
        const int64_t slot = p.window_slots[b];
        const int64_t rs = t % p.residual_len;
        const T* ring = reinterpret_cast<const T*>(p.window);
        lane_copy<T, E>(ring + (((slot * 2 + 0) * p.kv_heads + h) * p.residual_len + rs) * D + e0, kout);
        lane_copy<T, E>(ring + (((slot * 2 + 1) * p.kv_heads + h) * p.residual_len + rs) * D + e0, vout);
      } else {
#pragma unroll
        for (int j = 0; j < E; ++j) {
          kout[j] = ElemTraits<T>::from_float(0.0f);
          vout[j] = ElemTraits<T>::from_float(0.0f);
        }
      }
      continue;
    }
    const int64_t blk = t / p.block_size;
    const int tok = (int)(t % p.block_size);
    int32_t pid = -1;
    if (blk < p.max_blocks) pid = p.block_table[(int64_t)b * p.table_stride + blk];
    if (pid < 0 || pid >= p.num_pages) {
      if (dense_view) {  // the dense view has no holes: an unmapped block reads as zeros
#pragma unroll
        for (int j = 0; j < E; ++j) {
          kout[j] = ElemTraits<T>::from_float(0.0f);
          vout[j] = ElemTraits<T>::from_float(0.0f);
        }
      }
      continue;
    }
    const uint8_t* chunk = p.pages + ((int64_t)pid * p.kv_heads + h) * p.layout.chunk_bytes;

    // ---- keys: k_hat = norm / D * s1 * fwht( centroid[idx] + kappa * rnorm * s2 * fwht(2*sign - 1) ) ----------------
    const uint8_t* krow = chunk + p.layout.off_kcodes + tok * p.layout.key_bytes;
    float cent[E], sg[E];
    if constexpr (BITS == 4 && E == 4) {
      const uint32_t fields = reinterpret_cast<const uint16_t*>(krow)[lane];  // this lane's four nibbles
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const uint32_t field = (fields >> (4 * j)) & 0xFu;
        cent[j] = sm_cent[field & 7u];
        sg[j] = (field >> 3) ? 1.0f : -1.0f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const int d = e0 + j;
        uint32_t code, sbit;
        if constexpr (BITS == 4) {
          const uint32_t field = (krow[d >> 1] >> ((d & 1) * 4)) & 0xFu;
          code = field & 7u;
          sbit = field >> 3;
        } else if constexpr (BITS == 2) {
          const uint32_t field = (krow[d >> 2] >> ((d & 3) * 2)) & 3u;
          code = field & 1u;
          sbit = field >> 1;
        } else {
          code = (krow[d >> 2] >> ((d & 3) * 2)) & 3u;
          sbit = (krow[D / 4 + (d >> 3)] >> (d & 7)) & 1u;
        }
        cent[j] = sm_cent[code];
        sg[j] = sbit ? 1.0f : -1.0f;
      }
    }
    const float norm = reinterpret_cast<const float*>(chunk + p.layout.off_knorm)[tok];
    const float rnorm = reinterpret_cast<const float*>(chunk + p.layout.off_krnorm)[tok];
    warp_fwht<E>(sg, lane);
    const float coef = (1.2533141373155001f * rsqrt_dim_const<D>()) * rnorm;
#pragma unroll
    for (int j = 0; j < E; ++j) cent[j] = fmaf(coef, s2[j] < 0.0f ? -sg[j] : sg[j], cent[j]);
    warp_fwht<E>(cent, lane);
    const float scale = norm * (1.0f / (float)D);
    T kvals[E];
#pragma unroll
    for (int j = 0; j < E; ++j) kvals[j] = ElemTraits<T>::from_float(scale * (s1[j] < 0.0f ? -cent[j] : cent[j]));
    lane_copy<T, E>(kvals, kout);

    // ---- values: code * scale + zero --------------------------------------------------------------------------------
    const uint8_t* vrow = chunk + p.layout.off_vdata + tok * p.layout.value_bytes;
    const T* scales = reinterpret_cast<const T*>(chunk + p.layout.off_vscale) + tok * p.layout.groups;
    const T* zeros = reinterpret_cast<const T*>(chunk + p.layout.off_vzero) + tok * p.layout.groups;
    constexpr int kPerByte = 8 / VS;
    T vvals[E];
    if (p.value_group % E == 0) {  // one group per lane: its scale and zero point once
      const int g = e0 / p.value_group;
      const float v_scale = ElemTraits<T>::to_float(scales[g]), v_zero = ElemTraits<T>::to_float(zeros[g]);
      uint32_t codes = 0;
      if constexpr (E * VS == 16) codes = reinterpret_cast<const uint16_t*>(vrow)[lane];
      else if constexpr (E * VS == 8) codes = vrow[lane];
      else if constexpr (E * VS == 32) codes = reinterpret_cast<const uint32_t*>(vrow)[lane];
      else {
#pragma unroll
        for (int j = 0; j < E; ++j)
          codes |= ((vrow[(e0 + j) / kPerByte] >> (((e0 + j) % kPerByte) * VS)) & ((1u << VS) - 1u)) << (j * VS);
      }
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const uint32_t code = (codes >> (j * VS)) & ((1u << VS) - 1u);
        vvals[j] = ElemTraits<T>::from_float(__fadd_rn(__fmul_rn((float)code, v_scale), v_zero));
      }
    } else {
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const int d = e0 + j;
        const uint32_t code = (vrow[d / kPerByte] >> ((d % kPerByte) * VS)) & ((1u << VS) - 1u);
        const int g = d / p.value_group;
        const float prod = __fmul_rn((float)code, ElemTraits<T>::to_float(scales[g]));
        vvals[j] = ElemTraits<T>::from_float(__fadd_rn(prod, ElemTraits<T>::to_float(zeros[g])));
      }
    }
    lane_copy<T, E>(vvals, vout);
  }
}

}  // namespace anna

using namespace anna;

static int launch_materialize(TqMaterializeParams p, int batch, int kv_heads, int head_dim, int block_size, int bits,
                              int value_group, int dtype, cudaStream_t stream) {
  if (!tq_make_layout(head_dim, bits, block_size, dtype_bytes_of(dtype), value_group, &p.layout))
    return set_error(ANNA_ERR_INVALID, "TurboQuant materialize: unsupported geometry D=%d bits=%d S=%d group=%d", head_dim,
                     bits, block_size, value_group);
  const int64_t per_cta = (int64_t)kMaterializeWarps * kMaterializeTokens;
  dim3 grid((unsigned)((p.max_quantized_len + per_cta - 1) / per_cta), (unsigned)kv_heads, (unsigned)batch);
  return ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    return ANNA_DISPATCH_TQ_DIM(head_dim, D, [&]() -> int {
      return ANNA_DISPATCH_TQ_BITS(bits, BITS, [&]() -> int {
        tq_materialize_kernel<T, D, BITS><<<grid, kMaterializeWarps * 32, 0, stream>>>(p);
        return check_launch("tq_materialize_kernel");
      });
    });
  });
}

extern "C" int anna_tq_gather_dense(const uint8_t* packed_pages, const int32_t* block_table, int64_t table_stride,
                                    const void* window, const int64_t* window_slots, const int64_t* lengths,
                                    const float* signs1, const float* signs2, const float* centroids, void* key_out,
                                    void* value_out, int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t,
                                    int batch, int kv_heads, int head_dim, int block_size, int residual_len, int bits,
                                    int value_group, int64_t num_pages, int64_t max_blocks, int64_t max_len, int dtype,
                                    anna_stream_t stream) {
  ANNA_REQUIRE(window && window_slots && lengths && signs1 && signs2 && centroids && key_out && value_out,
               "anna_tq_gather_dense: null pointer argument");
  ANNA_REQUIRE(packed_pages != nullptr || num_pages == 0, "anna_tq_gather_dense: null page pool with num_pages > 0");
  ANNA_REQUIRE(block_table != nullptr || max_blocks == 0, "anna_tq_gather_dense: null block table with max_blocks > 0");
  ANNA_REQUIRE(batch > 0 && kv_heads > 0 && block_size >= 1 && residual_len >= 1 && max_len >= 0,
               "anna_tq_gather_dense: sizes must be positive");
  if (max_len == 0) return ANNA_OK;
  TqMaterializeParams p{};
  p.pages = packed_pages; p.block_table = block_table; p.table_stride = table_stride;
  p.signs1 = signs1; p.signs2 = signs2; p.centroids = centroids;
  p.key_out = key_out; p.value_out = value_out;
  p.out_stride_b = out_stride_b; p.out_stride_h = out_stride_h; p.out_stride_t = out_stride_t;
  p.kv_heads = kv_heads; p.block_size = block_size; p.value_group = value_group;
  p.num_pages = num_pages; p.max_blocks = max_blocks; p.max_quantized_len = max_len;
  p.window = window; p.window_slots = window_slots; p.lengths = lengths; p.residual_len = residual_len;
  return launch_materialize(p, batch, kv_heads, head_dim, block_size, bits, value_group, dtype, (cudaStream_t)stream);
}

extern "C" int anna_tq_materialize(const uint8_t* packed_pages, const int32_t* block_table, int64_t table_stride,
                                   const int64_t* quantized_lengths, const float* signs1, const float* signs2,
                                   const float* centroids, void* key_out, void* value_out, int64_t out_stride_b,
                                   int64_t out_stride_h, int64_t out_stride_t, int batch, int kv_heads, int head_dim,
                                   int block_size, int bits, int value_group, int64_t num_pages, int64_t max_blocks,
                                   int64_t max_quantized_len, int dtype, anna_stream_t stream) {
  ANNA_REQUIRE(packed_pages && block_table && quantized_lengths && signs1 && signs2 && centroids && key_out && value_out,
               "anna_tq_materialize: null pointer argument");
  ANNA_REQUIRE(batch > 0 && kv_heads > 0 && block_size >= 1 && max_quantized_len >= 0,
               "anna_tq_materialize: sizes must be positive");
  if (max_quantized_len == 0) return ANNA_OK;
  TqMaterializeParams p{};
  p.pages = packed_pages; p.block_table = block_table; p.table_stride = table_stride;
  p.quantized_lengths = quantized_lengths; p.signs1 = signs1; p.signs2 = signs2; p.centroids = centroids;
  p.key_out = key_out; p.value_out = value_out;
  p.out_stride_b = out_stride_b; p.out_stride_h = out_stride_h; p.out_stride_t = out_stride_t;
  p.kv_heads = kv_heads; p.block_size = block_size; p.value_group = value_group;
  p.num_pages = num_pages; p.max_blocks = max_blocks; p.max_quantized_len = max_quantized_len;
  return launch_materialize(p, batch, kv_heads, head_dim, block_size, bits, value_group, dtype, (cudaStream_t)stream);
}
