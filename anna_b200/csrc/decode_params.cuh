// Parameters shared by the CUDA-core and tensor-core split kernels for un-quantized K/V.
#pragma once

#include "common.cuh"
#include "fused_combine.cuh"

namespace anna {

struct DenseDecodeParams {
  const void* q;
  int64_t q_stride_b, q_stride_h;
  const void* key;
  const void* value;
  // paged addressing (page_table != nullptr): element offset = page_id * page_stride + (t % S) * D
  const int32_t* page_table;
  int64_t table_stride;
  int64_t page_stride;
  int64_t num_pages;
  int block_size;
  int block_shift;  // log2(block_size) when it is a power of two, else -1
  // dense addressing: element offset = b * kv_stride_b + h * kv_stride_h + t * kv_stride_t
  int64_t kv_stride_b, kv_stride_h, kv_stride_t;
  int ring_len;  // > 0: token t sits at (t % ring_len) * head_dim (window ring of a TurboQuant row)
  const int64_t* visible_lengths;  // may be null in dense mode: all `max_len` keys visible
  int64_t max_len;
  float* stats;
  float* values;
  int q_heads, kv_heads, groups;
  int chunk_tokens, num_chunks, chunk_capacity;
  float scaling;
  FusedCombine fused;  // fused.counters == nullptr: partials only, a second pass merges them
};

// Tensor-core split pass (paged_decode_mma.cu): 16-bit dtypes, head_dim 64 / 128 / 256.
bool dense_split_mma_applicable(const DenseDecodeParams& p, int head_dim, int dtype);
int launch_dense_split_mma(const DenseDecodeParams& p, int batch, int head_dim, int dtype, cudaStream_t stream);
// one resident wave with an even share of tiles per CTA; needs the fused merge and the library's own split plan
bool dense_balanced_mma_applicable(const DenseDecodeParams& p, int batch);
int launch_dense_balanced_mma(const DenseDecodeParams& p, int batch, int head_dim, int dtype, cudaStream_t stream);

}  // namespace anna
