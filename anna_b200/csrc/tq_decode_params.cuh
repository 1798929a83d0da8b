// Parameters of the TurboQuant decode split kernels (CUDA-core and tensor-core).
#pragma once

#include "common.cuh"
#include "fused_combine.cuh"

namespace anna {

struct TqDecodeParams {
  const void* q;
  int64_t q_stride_b, q_stride_h;
  const uint8_t* pages;
  const int32_t* block_table;
  int64_t table_stride;
  const void* window;
  const int64_t* window_slots;
  const int64_t* lengths;
  const float* signs1;
  const float* signs2;
  const float* centroids;
  float* stats;
  float* values;
  int q_heads, kv_heads, groups;
  int block_size, residual_len, value_group;
  int block_shift;  // log2(block_size) when it is a power of two, else -1
  int64_t num_pages, max_blocks, max_len;
  int chunk_tokens, num_chunks, chunk_capacity;
  int num_window_chunks;  // split-K slots [0, num_window_chunks) cover the window ring, the rest the packed prefix
  float scaling;
  anna_tq_layout layout;
  FusedCombine fused;
  void* query_frags;  // scratch for the rotated fp16 query fragments (tensor-core path), or nullptr
};

// Tensor-memory split pass (tq_decode_umma.cu): 16-bit cache dtypes, head_dim 128, 3- / 4-bit codes, 16-token pages,
// value group 32, at most 4 query heads per kv head.
bool tq_split_umma_applicable(const TqDecodeParams& p, int head_dim, int bits, int dtype);
int launch_tq_split_umma(const TqDecodeParams& p, int batch, int bits, int dtype, cudaStream_t stream);
int tq_decode_umma_faults(int* count);
size_t tq_umma_query_bytes();  // query operand image per (row, kv head) of that path
// the window-ring launch of the tensor-core paths (tq_decode_mma.cu)
int launch_tq_window_split(const TqDecodeParams& p, int batch, int head_dim, int dtype, cudaStream_t stream);

// Bytes of query scratch the tensor-core paths need per call: 32 * head_dim fragment bytes per (row, kv head, group of
// 8 query heads) for the mma.sync path, one query operand image per (row, kv head) for the tensor-memory path.
inline size_t tq_query_scratch_bytes(int batch, int q_heads, int kv_heads, int head_dim) {
  const size_t units = (size_t)batch * kv_heads * ((q_heads / kv_heads + 7) / 8);
  const size_t frag = (size_t)32 * head_dim;
  const size_t image = tq_umma_query_bytes();
  return units * (frag > image ? frag : image);
}

// Tensor-core split pass (tq_decode_mma.cu): 16-bit cache dtypes, head_dim 128 / 256, value group 32, page size % 16 == 0.
bool tq_split_mma_applicable(const TqDecodeParams& p, int head_dim, int dtype);
int launch_tq_split_mma(const TqDecodeParams& p, int batch, int head_dim, int bits, int dtype, cudaStream_t stream);

// bounded copy waits that expired in the tensor-core packed decode on the current device (tq_decode_mma.cu)
int tq_decode_mma_faults(int* count);

}  // namespace anna
