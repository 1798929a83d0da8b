// Paged GQA decode for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc themselves: a plugin that is handed raw device pointers
// by an engine that owns the memory pool and forbids foreign allocations (an allocation behind the pool's back would
// break its accounting or its capture rules), or a component that runs where the allocator is locked.  Those callers
// can pass inputs and outputs but have nowhere to put the split-K scratch that anna_paged_gqa_decode asks for.  This
// entry point brings its own: a fixed array inside the library's device image.
#include "common.cuh"

namespace anna {

// 16 MiB per GPU that loads the library, held until the process exits.
constexpr size_t kNoAllocScratchBytes = 16u << 20;
constexpr size_t kNoAllocCounterBytes = 64u << 10;  // head of the array: arrival counters of the in-kernel merge

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of the array above, per device ordinal.  The array's name is only a handle on the host: the address
// a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.  The table is
// filled without a lock: host threads that make their first call on one device at the same time may each do the
// look-up, and all of them store the same address.
static void* g_noalloc_scratch_ptr[64] = {};

static int noalloc_scratch_base(unsigned char** base) {
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64) return set_error(ANNA_ERR_UNSUPPORTED, "device ordinal %d is out of range", device);
  if (g_noalloc_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    ANNA_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) return set_error(ANNA_ERR_CUDA, "cudaGetSymbolAddress returned a null scratch address");
    g_noalloc_scratch_ptr[device] = ptr;
  }
  *base = static_cast<unsigned char*>(g_noalloc_scratch_ptr[device]);
  return ANNA_OK;
}

}  // namespace anna

using namespace anna;

extern "C" size_t anna_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int anna_paged_gqa_decode_noalloc(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                             const void* key_pages, const void* value_pages,
                                             const int32_t* page_table, int64_t table_stride,
                                             const int64_t* visible_lengths, const void* gate, int64_t gate_stride_b,
                                             int64_t gate_stride_h, void* out, int64_t out_stride_b,
                                             int64_t out_stride_h, int batch, int q_heads, int kv_heads, int head_dim,
                                             int block_size, int64_t num_pages, int64_t max_blocks, float scaling,
                                             int dtype, anna_stream_t stream) {
  ANNA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && head_dim > 0 && block_size > 0 &&
                   max_blocks > 0,
               "anna_paged_gqa_decode_noalloc: sizes must be positive and query heads a multiple of kv heads");
  int chunk_tokens = 0, num_chunks = 0;
  int rc = anna_decode_plan(batch, kv_heads, max_blocks * (int64_t)block_size, &chunk_tokens, &num_chunks);
  if (rc != ANNA_OK) return rc;
  const size_t group_tiles = (size_t)(q_heads / kv_heads + 7) / 8;
  const size_t counter_bytes = 2 * sizeof(int32_t) * (size_t)batch * kv_heads * group_tiles;  // arrivals + cursors
  const size_t heads = (size_t)batch * q_heads;
  const size_t stats_bytes = sizeof(float) * heads * num_chunks * 2;
  const size_t values_bytes = sizeof(float) * heads * num_chunks * head_dim;
  const size_t stats_offset = kNoAllocCounterBytes;
  const size_t values_offset = (stats_offset + stats_bytes + 255) / 256 * 256;
  if (counter_bytes > kNoAllocCounterBytes)
    return set_error(ANNA_ERR_WORKSPACE,
                     "anna_paged_gqa_decode_noalloc: batch * kv_heads * ceil(G / 8) = %zu (row, head-group) pairs need "
                     "%zu bytes of merge counters but the built-in array reserves %zu (at most %zu pairs); use "
                     "anna_paged_gqa_decode with caller-provided scratch",
                     (size_t)batch * kv_heads * group_tiles, counter_bytes, (size_t)kNoAllocCounterBytes,
                     (size_t)(kNoAllocCounterBytes / (2 * sizeof(int32_t))));
  if (values_offset + values_bytes > kNoAllocScratchBytes)
    return set_error(ANNA_ERR_WORKSPACE,
                     "anna_paged_gqa_decode_noalloc: this problem needs %zu bytes of split-K scratch but the built-in "
                     "array holds %zu; use anna_paged_gqa_decode with caller-provided scratch",
                     values_offset + values_bytes, (size_t)kNoAllocScratchBytes);
  unsigned char* base = nullptr;
  rc = noalloc_scratch_base(&base);
  if (rc != ANNA_OK) return rc;
  // The array keeps whatever the previous call left behind.  Partials are fully rewritten before they are read, but
  // the arrival counters must start at zero, so that region is cleared on the caller's stream first.
  ANNA_CUDA_CHECK(cudaMemsetAsync(base, 0, counter_bytes, (cudaStream_t)stream));
  return anna_paged_gqa_decode(q, q_stride_b, q_stride_h, key_pages, value_pages, page_table, table_stride,
                               visible_lengths, gate, gate_stride_b, gate_stride_h, out, out_stride_b, out_stride_h,
                               reinterpret_cast<float*>(base + stats_offset),
                               reinterpret_cast<float*>(base + values_offset), num_chunks, 0,
                               reinterpret_cast<int32_t*>(base), batch, q_heads, kv_heads, head_dim, block_size,
                               num_pages, max_blocks, scaling, dtype, stream);
}
