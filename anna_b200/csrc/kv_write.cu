// Paged write of new un-quantized K/V tokens (batched page scatter).
#include "common.cuh"

namespace anna {

struct KvWriteParams {
  const void* k_new;
  const void* v_new;
  int64_t stride_b, stride_h, stride_t;
  void* key_pages;
  void* value_pages;
  const int32_t* page_table;
  int64_t table_stride;
  const int64_t* past_lengths;
  int64_t* new_lengths;
  int batch, kv_heads, new_tokens, head_dim, block_size;
  int64_t num_pages, max_blocks;
  int32_t* status;
};

// One thread moves one 16-byte piece of K and the matching piece of V.
template <typename T>
__global__ void __launch_bounds__(256) paged_kv_write_kernel(const KvWriteParams p) {
  constexpr int kVec = ElemTraits<T>::kVec;
  const int pieces = p.head_dim / kVec;
  const int64_t total = (int64_t)p.batch * p.kv_heads * p.new_tokens * pieces;
  for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < total;
       item += (int64_t)gridDim.x * blockDim.x) {
    const int piece = (int)(item % pieces);
    int64_t rest = item / pieces;
    const int t = (int)(rest % p.new_tokens);
    rest /= p.new_tokens;
    const int h = (int)(rest % p.kv_heads);
    const int b = (int)(rest / p.kv_heads);
    const int64_t past = p.past_lengths[b];
    if (p.new_lengths != nullptr && (piece | t | h) == 0) p.new_lengths[b] = past + p.new_tokens;
    const int64_t pos = past + t;
    const int64_t blk = pos / p.block_size;
    const int slot = (int)(pos % p.block_size);
    int32_t pid = -1;
    if (blk < p.max_blocks) pid = p.page_table[(int64_t)b * p.table_stride + blk];
    if (pid < 0 || pid >= p.num_pages) {
      if (p.status) atomicOr(p.status, (int)ANNA_DEV_BAD_PAGE);
      continue;
    }
    const int64_t src = (int64_t)b * p.stride_b + (int64_t)h * p.stride_h + (int64_t)t * p.stride_t + piece * kVec;
    const int64_t dst = (((int64_t)pid * p.kv_heads + h) * p.block_size + slot) * p.head_dim + piece * kVec;
    const uint4 kv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.k_new) + src);
    const uint4 vv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.v_new) + src);
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.key_pages) + dst) = kv;
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.value_pages) + dst) = vv;
  }
}

// Block-table patch: entry i is the triple (row, column, page id).
__global__ void block_table_patch_kernel(int32_t* table, int64_t table_stride, int64_t rows, int64_t cols,
                                         const int32_t* entries, int count) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
    const int32_t row = entries[3 * i], col = entries[3 * i + 1];
    if (row >= 0 && row < rows && col >= 0 && col < cols) table[(int64_t)row * table_stride + col] = entries[3 * i + 2];
  }
}

struct KvGatherParams {
  const void* key_pages;
  const void* value_pages;
  const int32_t* page_table;
  int64_t table_stride;
  const int64_t* lengths;
  void* key_out;
  void* value_out;
  int64_t out_stride_b, out_stride_h, out_stride_t;
  int batch, kv_heads, head_dim, block_size;
  int64_t num_pages, max_blocks, max_len;
};

// Dense view of paged K/V: one thread moves one 16-byte piece of K and the matching piece of V; positions at or past
// a row's length, and tokens of unmapped blocks, are written as zeros.
template <typename T>
__global__ void __launch_bounds__(256) paged_kv_gather_kernel(const KvGatherParams p) {
  constexpr int kVec = ElemTraits<T>::kVec;
  const int pieces = p.head_dim / kVec;
  const int64_t total = (int64_t)p.batch * p.kv_heads * p.max_len * pieces;
  for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < total;
       item += (int64_t)gridDim.x * blockDim.x) {
    const int piece = (int)(item % pieces);
    int64_t rest = item / pieces;
    const int64_t t = rest % p.max_len;
    rest /= p.max_len;
    const int h = (int)(rest % p.kv_heads);
    const int b = (int)(rest / p.kv_heads);
    uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = kv;
    if (t < p.lengths[b]) {
      const int64_t blk = t / p.block_size;
      const int slot = (int)(t % p.block_size);
      const int32_t pid = blk < p.max_blocks ? p.page_table[(int64_t)b * p.table_stride + blk] : -1;
      if (pid >= 0 && pid < p.num_pages) {
        const int64_t src = (((int64_t)pid * p.kv_heads + h) * p.block_size + slot) * p.head_dim + piece * kVec;
        kv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.key_pages) + src);
        vv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.value_pages) + src);
      }
    }
    const int64_t dst = (int64_t)b * p.out_stride_b + (int64_t)h * p.out_stride_h + t * p.out_stride_t + piece * kVec;
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.key_out) + dst) = kv;
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.value_out) + dst) = vv;
  }
}

}  // namespace anna

using namespace anna;

extern "C" int anna_block_table_patch(int32_t* table, int64_t table_stride, int64_t rows, int64_t cols,
                                      const int32_t* entries, int count, anna_stream_t stream) {
  ANNA_REQUIRE(table != nullptr && entries != nullptr, "anna_block_table_patch: null pointer argument");
  ANNA_REQUIRE(rows > 0 && cols > 0 && table_stride >= cols && count >= 0, "anna_block_table_patch: bad geometry");
  if (count == 0) return ANNA_OK;
  int blocks = (count + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  block_table_patch_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(table, table_stride, rows, cols, entries, count);
  return check_launch("block_table_patch_kernel");
}

extern "C" int anna_paged_kv_gather(const void* key_pages, const void* value_pages, const int32_t* page_table,
                                    int64_t table_stride, const int64_t* lengths, void* key_out, void* value_out,
                                    int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t, int batch,
                                    int kv_heads, int head_dim, int block_size, int64_t num_pages, int64_t max_blocks,
                                    int64_t max_len, int dtype, anna_stream_t stream) {
  ANNA_REQUIRE(key_pages && value_pages && page_table && lengths && key_out && value_out,
               "anna_paged_kv_gather: null pointer argument");
  ANNA_REQUIRE(batch > 0 && kv_heads > 0 && block_size > 0 && num_pages > 0 && max_blocks > 0 && max_len > 0,
               "anna_paged_kv_gather: sizes must be positive");
  const int vec = dtype == ANNA_DTYPE_F32 ? 4 : 8;
  ANNA_REQUIRE(head_dim > 0 && head_dim % vec == 0, "anna_paged_kv_gather: head_dim %d must be a multiple of %d",
               head_dim, vec);
  ANNA_REQUIRE(out_stride_b % vec == 0 && out_stride_h % vec == 0 && out_stride_t % vec == 0,
               "anna_paged_kv_gather: output strides must keep rows 16-byte aligned");
  KvGatherParams p{key_pages, value_pages, page_table, table_stride, lengths, key_out, value_out, out_stride_b,
                   out_stride_h, out_stride_t, batch, kv_heads, head_dim, block_size, num_pages, max_blocks, max_len};
  const int64_t total = (int64_t)batch * kv_heads * max_len * (head_dim / vec);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    paged_kv_gather_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    return check_launch("paged_kv_gather_kernel");
  });
}

extern "C" int anna_paged_kv_write(const void* k_new, const void* v_new, int64_t kn_stride_b, int64_t kn_stride_h,
                                   int64_t kn_stride_t, void* key_pages, void* value_pages,
                                   const int32_t* page_table, int64_t table_stride, const int64_t* past_lengths,
                                   int64_t* new_lengths, int batch, int kv_heads, int new_tokens, int head_dim, int block_size,
                                   int64_t num_pages, int64_t max_blocks, int dtype, int32_t* status,
                                   anna_stream_t stream) {
  ANNA_REQUIRE(k_new && v_new && key_pages && value_pages && page_table && past_lengths,
               "anna_paged_kv_write: null pointer argument");
  ANNA_REQUIRE(new_lengths != past_lengths, "anna_paged_kv_write: new_lengths must not alias past_lengths");
  ANNA_REQUIRE(batch > 0 && kv_heads > 0 && new_tokens > 0 && block_size > 0 && num_pages > 0 && max_blocks > 0,
               "anna_paged_kv_write: sizes must be positive");
  const int vec = dtype == ANNA_DTYPE_F32 ? 4 : 8;
  ANNA_REQUIRE(head_dim > 0 && head_dim % vec == 0, "anna_paged_kv_write: head_dim %d must be a multiple of %d",
               head_dim, vec);
  ANNA_REQUIRE(kn_stride_b % vec == 0 && kn_stride_h % vec == 0 && kn_stride_t % vec == 0,
               "anna_paged_kv_write: source strides must keep rows 16-byte aligned");
  KvWriteParams p{k_new, v_new, kn_stride_b, kn_stride_h, kn_stride_t, key_pages, value_pages, page_table,
                  table_stride, past_lengths, new_lengths, batch, kv_heads, new_tokens, head_dim, block_size, num_pages,
                  max_blocks, status};
  const int64_t total = (int64_t)batch * kv_heads * new_tokens * (head_dim / vec);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    paged_kv_write_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    return check_launch("paged_kv_write_kernel");
  });
}
