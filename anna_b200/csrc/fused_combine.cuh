// Split-K merge done by the last CTA that finishes a (row, kv-head group): no second launch, no waiting.
//
// Every CTA of the split pass publishes its partial, fences, and bumps a per-(row, group) counter.  The CTA that
// observes the final count owns the merge: it re-reads the partials (L2 resident), applies the optional sigmoid(gate)
// epilogue and stores the output row.  Nobody spins: a CTA either is last or leaves.  The counter is reset by the
// merging CTA, so the caller's buffer stays all-zero between launches.
#pragma once

#include "common.cuh"

namespace anna {

struct FusedCombine {
  int32_t* counters;   // [batch, kv heads x groups-of-8] zero on entry; nullptr selects the two-pass path
  void* out;
  int64_t out_stride_b, out_stride_h;
  const void* gate;
  int64_t gate_stride_b, gate_stride_h;
  // KV-head-sharded decode: the same rows of the output tensors of the other ranks (peer memory mapped into this
  // process).  Every merged output row is stored to all of them at the offset it has in `out`.
  void* peers[kMaxPeerOutputs];
  int num_peers;
};

constexpr int kFusedMaxChunks = 512;  // weights of one head are staged in shared memory

// Called by all threads of the CTA after they wrote their partial.  `active_chunks` = partials that contribute to this
// (row, group), whose arrivals are counted in counters[counter_index]; stats / values point at chunk 0 of query head
// hq0.  Natural-log stats.  THREADS = blockDim.x.
template <typename T, int D, int THREADS>
__device__ __forceinline__ void fused_combine_tail(const FusedCombine& fc, int b, int hq0, int g_count,
                                                   int active_chunks, int chunk_capacity, const float* stats,
                                                   const float* values, float* smem_weights /* [8][kFusedMaxChunks] */,
                                                   int64_t counter_index) {
  __shared__ int s_is_last;
  __syncthreads();  // all partial stores of this CTA are ordered before the fence below
  if (threadIdx.x == 0) {
    __threadfence();
    int32_t* counter = fc.counters + counter_index;
    const int prev = atomicAdd(counter, 1);
    s_is_last = (prev == active_chunks - 1) ? 1 : 0;
    if (s_is_last) *counter = 0;
  }
  __syncthreads();
  if (!s_is_last) return;
  __threadfence();

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  constexpr int kWarps = THREADS / 32;
  // one warp per head: max, denominator, normalised weights
  for (int g = warp; g < g_count; g += kWarps) {
    const float* st = stats + (int64_t)g * chunk_capacity * 2;
    float m = -INFINITY;
    for (int c = lane; c < active_chunks; c += 32) m = fmaxf(m, __ldcg(st + 2 * c));
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    const float m_ref = m == -INFINITY ? 0.0f : m;
    float den = 0.0f;
    for (int c = lane; c < active_chunks; c += 32) {
      const float w = __expf(__ldcg(st + 2 * c) - m_ref);
      den += __ldcg(st + 2 * c + 1) * w;
      smem_weights[g * kFusedMaxChunks + c] = w;
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) den += __shfl_xor_sync(0xffffffffu, den, d);
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    for (int c = lane; c < active_chunks; c += 32) smem_weights[g * kFusedMaxChunks + c] *= inv;
  }
  __syncthreads();
  for (int item = threadIdx.x; item < g_count * D; item += THREADS) {
    const int g = item / D;
    const int d = item % D;
    const float* vals = values + (int64_t)g * chunk_capacity * D + d;
    const float* w = smem_weights + g * kFusedMaxChunks;
    float acc = 0.0f;
    for (int c = 0; c < active_chunks; ++c) acc = fmaf(__ldcg(vals + (int64_t)c * D), w[c], acc);
    if (fc.gate) {
      const T* gate = reinterpret_cast<const T*>(fc.gate) + (int64_t)b * fc.gate_stride_b +
                      (int64_t)(hq0 + g) * fc.gate_stride_h;
      acc *= sigmoidf_fast(ElemTraits<T>::to_float(gate[d]));
    }
    const int64_t offset = (int64_t)b * fc.out_stride_b + (int64_t)(hq0 + g) * fc.out_stride_h + d;
    const T result = ElemTraits<T>::from_float(acc);
    reinterpret_cast<T*>(fc.out)[offset] = result;
    for (int peer = 0; peer < fc.num_peers; ++peer) reinterpret_cast<T*>(fc.peers[peer])[offset] = result;
  }
  // stores to other GPUs are ordered before whatever this stream signals to them after the kernel
  if (fc.num_peers > 0) __threadfence_system();
}

// A row with no visible key has no contributing CTA; the CTA of chunk 0 writes its zeros.
template <typename T, int D, int THREADS>
__device__ __forceinline__ void fused_write_zero_row(const FusedCombine& fc, int b, int hq0, int g_count) {
  for (int item = threadIdx.x; item < g_count * D; item += THREADS) {
    const int g = item / D;
    const int d = item % D;
    const int64_t offset = (int64_t)b * fc.out_stride_b + (int64_t)(hq0 + g) * fc.out_stride_h + d;
    reinterpret_cast<T*>(fc.out)[offset] = ElemTraits<T>::from_float(0.0f);
    for (int peer = 0; peer < fc.num_peers; ++peer)
      reinterpret_cast<T*>(fc.peers[peer])[offset] = ElemTraits<T>::from_float(0.0f);
  }
  if (fc.num_peers > 0) __threadfence_system();
}

}  // namespace anna
