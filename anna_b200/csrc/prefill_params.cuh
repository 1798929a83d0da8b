// Arguments of the multi-token attention kernels (gqa_prefill.cu: mma.sync; gqa_prefill_umma.cu: tcgen05).
#pragma once

#include "common.cuh"

namespace anna {

struct PrefillParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  const int64_t* key_lengths;
  int64_t q_stride_b, q_stride_h, q_stride_t;
  int64_t kv_stride_b, kv_stride_h, kv_stride_t;
  int64_t out_stride_b, out_stride_h, out_stride_t;
  int q_len, groups, causal;
  int64_t key_len;
  float scale_log2;  // scaling * log2(e)
};

constexpr int kPrefillNotServed = -1;  // launch_prefill_umma: the caller should use the mma.sync kernel instead

// true when the tensor-memory kernel serves this problem (head_dim 128, 16-bit, not switched off)
bool prefill_umma_applicable(const PrefillParams& p, int head_dim, int dtype);
int launch_prefill_umma(const PrefillParams& p, int batch, int q_heads, int head_dim, int dtype, cudaStream_t stream);
int prefill_umma_faults(int* count);

}  // namespace anna
