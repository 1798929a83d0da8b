// Single-token GQA decode over un-quantized K/V: paged pools or dense strided tensors.
#include "decode_core.cuh"
#include "decode_params.cuh"

namespace anna {

template <typename T, int D, int G>
__global__ void __launch_bounds__(kDecodeThreads)
dense_decode_split_kernel(const DenseDecodeParams p) {
  using Cfg = DecodeCfg<T, D, G>;
  extern __shared__ float smem[];
  const int chunk = blockIdx.x;
  const int group_tiles = (p.groups + G - 1) / G;
  const int kvh = blockIdx.y / group_tiles;
  const int g0 = (blockIdx.y % group_tiles) * G;
  const int g_count = min(G, p.groups - g0);
  const int b = blockIdx.z;

  int64_t len = p.visible_lengths ? p.visible_lengths[b] : p.max_len;
  len = max((int64_t)0, min(len, p.max_len));
  const int64_t t0 = (int64_t)chunk * p.chunk_tokens;
  if (t0 >= len) return;
  const int64_t t1 = min(len, t0 + p.chunk_tokens);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int sub = lane / Cfg::kLpt;
  const int dl = lane % Cfg::kLpt;
  const int hq0 = kvh * p.groups + g0;

  // stage the group's queries in shared memory as float
  float* q_smem = smem;  // [G][D]
  const T* q_ptr = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b;
  for (int item = threadIdx.x; item < G * D; item += kDecodeThreads) {
    const int g = item / D;
    const int d = item % D;
    q_smem[item] = g < g_count ? ElemTraits<T>::to_float(q_ptr[(int64_t)(hq0 + g) * p.q_stride_h + d]) : 0.0f;
  }
  __syncthreads();

  TeamState<T, D, G> st;
  st.reset();
  load_query_from_smem<T, D, G>(st, q_smem, dl, p.scaling);
  __syncthreads();  // q_smem is reused by the merge below

  const bool paged = p.page_table != nullptr;
  const T* k_base;
  const T* v_base;
  if (paged) {
    const int64_t head_off = (int64_t)kvh * p.block_size * D;
    k_base = reinterpret_cast<const T*>(p.key) + head_off;
    v_base = reinterpret_cast<const T*>(p.value) + head_off;
  } else {
    const int64_t head_off = (int64_t)b * p.kv_stride_b + (int64_t)kvh * p.kv_stride_h;
    k_base = reinterpret_cast<const T*>(p.key) + head_off;
    v_base = reinterpret_cast<const T*>(p.value) + head_off;
  }
  const int32_t* table_row = paged ? p.page_table + (int64_t)b * p.table_stride : nullptr;

  constexpr int kStep = kDecodeWarps * Cfg::kTpw * kUnroll;  // tokens per CTA iteration
  for (int64_t base = t0 + warp * (Cfg::kTpw * kUnroll); base < t1; base += kStep) {
    int64_t off[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t t = base + u * Cfg::kTpw + sub;
      off[u] = -1;
      if (t < t1) {
        if (paged) {
          const int32_t pid = table_row[t / p.block_size];
          if (pid >= 0 && pid < p.num_pages) off[u] = (int64_t)pid * p.page_stride + (t % p.block_size) * D;
        } else {
          off[u] = t * p.kv_stride_t;
        }
      }
    }
    team_consume<T, D, G>(st, k_base, v_base, off, dl);
  }

  const int64_t part = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity + chunk;
  cta_merge_store<T, D, G>(st, smem, warp, sub, dl, g_count, p.stats + part * 2, p.values + part * D,
                           (int64_t)p.chunk_capacity * 2, (int64_t)p.chunk_capacity * D);
}

template <typename T, int D, int G>
static int launch_dense_split(const DenseDecodeParams& p, int batch, cudaStream_t stream) {
  using Cfg = DecodeCfg<T, D, G>;
  const size_t smem_merge = sizeof(float) * (size_t)Cfg::kTeams * G * (D + 2);
  const size_t smem_q = sizeof(float) * (size_t)G * D;
  const size_t smem = smem_merge > smem_q ? smem_merge : smem_q;
  auto kernel = dense_decode_split_kernel<T, D, G>;
  if (smem > 48 * 1024) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const int group_tiles = (p.groups + G - 1) / G;
  dim3 grid((unsigned)p.num_chunks, (unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
  kernel<<<grid, kDecodeThreads, smem, stream>>>(p);
  return check_launch("dense_decode_split_kernel");
}

static int run_dense_decode(DenseDecodeParams p, const void* gate, int64_t gate_stride_b, int64_t gate_stride_h,
                            void* out, int64_t out_stride_b, int64_t out_stride_h, float* partial_stats,
                            float* partial_values, int chunk_capacity, int chunk_tokens_in, int32_t* split_counters,
                            int batch, int head_dim, int dtype, cudaStream_t stream) {
  int chunk_tokens = 0, num_chunks = 0;
  int rc = resolve_split(batch, p.kv_heads, p.max_len, chunk_tokens_in, chunk_capacity, partial_stats, partial_values,
                         &chunk_tokens, &num_chunks);
  if (rc != ANNA_OK) return rc;
  SplitWorkspace ws{partial_stats, partial_values, chunk_capacity};
  p.stats = ws.stats;
  p.values = ws.values;
  p.chunk_tokens = chunk_tokens;
  p.num_chunks = num_chunks;
  p.chunk_capacity = chunk_capacity;
  if (dense_split_mma_applicable(p, head_dim, dtype)) {
    if (split_counters != nullptr && num_chunks <= kFusedMaxChunks) {
      p.fused = FusedCombine{split_counters, out, out_stride_b, out_stride_h, gate, gate_stride_b, gate_stride_h};
      if (chunk_tokens_in <= 0) {
        // Two schedules for the same tile body.  Few CTAs' worth of work: one resident wave with an even share per CTA
        // (no tail, one pipeline start per CTA).  Many: fixed chunks handed out by the hardware block scheduler, which
        // lets faster SMs take more chunks; measured 3-10 % ahead from about 6000 grid CTAs on (48+ rows of 1-8 K
        // tokens, 32+ rows of 16-32 K), and up to 40 % behind below that.
        const int64_t grid_ctas = (int64_t)num_chunks * p.kv_heads * ((p.groups + 7) / 8) * batch;
        if (grid_ctas < 6000 && dense_balanced_mma_applicable(p, batch))
          return launch_dense_balanced_mma(p, batch, head_dim, dtype, stream);
      }
      return launch_dense_split_mma(p, batch, head_dim, dtype, stream);
    }
    rc = launch_dense_split_mma(p, batch, head_dim, dtype, stream);
  } else {
    const int gpad = padded_group(p.groups);
    rc = ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
      return ANNA_DISPATCH_DIM(head_dim, D, [&]() -> int {
        return ANNA_DISPATCH_GROUP(gpad, G, [&]() -> int { return launch_dense_split<T, D, G>(p, batch, stream); });
      });
    });
  }
  if (rc != ANNA_OK) return rc;
  return launch_split_combine(ws, nullptr, p.visible_lengths, p.visible_lengths ? -1 : p.max_len, p.max_len, 0, gate,
                              gate_stride_b, gate_stride_h, out, out_stride_b, out_stride_h, batch, p.q_heads,
                              head_dim, chunk_tokens, num_chunks, dtype, stream);
}

}  // namespace anna

using namespace anna;

extern "C" int anna_decode_plan(int batch, int kv_heads, int64_t max_len, int* chunk_tokens, int* num_chunks) {
  ANNA_REQUIRE(batch > 0 && kv_heads > 0 && max_len >= 0, "anna_decode_plan: batch, kv_heads must be positive");
  ANNA_REQUIRE(chunk_tokens != nullptr && num_chunks != nullptr, "anna_decode_plan: null output pointer");
  // Aim for a few thousand CTAs (148 SMs x several resident CTAs x a few waves) without dropping below 64 tokens
  // or going above 1024 tokens per CTA.
  const int64_t streams = (int64_t)batch * kv_heads;
  const int64_t target_ctas = 148 * 24;
  int64_t want_chunks = (target_ctas + streams - 1) / streams;
  if (want_chunks < 1) want_chunks = 1;
  int64_t chunk = 1024;
  while (chunk > 64 && (max_len + chunk - 1) / chunk < want_chunks) chunk >>= 1;
  int64_t chunks = (max_len + chunk - 1) / chunk;
  if (chunks < 1) chunks = 1;
  ANNA_REQUIRE(chunks <= 65535 * 16, "anna_decode_plan: context of %lld tokens is too long", (long long)max_len);
  *chunk_tokens = (int)chunk;
  *num_chunks = (int)chunks;
  return ANNA_OK;
}


extern "C" int anna_paged_gqa_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* key_pages,
                                     const void* value_pages, const int32_t* page_table, int64_t table_stride,
                                     const int64_t* visible_lengths, const void* gate, int64_t gate_stride_b,
                                     int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h,
                                     float* partial_stats, float* partial_values, int chunk_capacity,
                                     int chunk_tokens, int32_t* split_counters, int batch, int q_heads, int kv_heads,
                                     int head_dim,
                                     int block_size, int64_t num_pages, int64_t max_blocks, float scaling, int dtype,
                                     anna_stream_t stream) {
  ANNA_REQUIRE(q && key_pages && value_pages && page_table && visible_lengths && out,
               "anna_paged_gqa_decode: null pointer argument");
  ANNA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
               "anna_paged_gqa_decode: query heads (%d) must be a positive multiple of kv heads (%d)", q_heads, kv_heads);
  ANNA_REQUIRE(block_size >= 1 && num_pages >= 1 && max_blocks >= 1 && table_stride >= max_blocks,
               "anna_paged_gqa_decode: bad paging geometry (block_size=%d pages=%lld max_blocks=%lld stride=%lld)",
               block_size, (long long)num_pages, (long long)max_blocks, (long long)table_stride);
  DenseDecodeParams p{};
  p.q = q; p.q_stride_b = q_stride_b; p.q_stride_h = q_stride_h;
  p.key = key_pages; p.value = value_pages;
  p.page_table = page_table; p.table_stride = table_stride;
  p.page_stride = (int64_t)kv_heads * block_size * head_dim;
  p.num_pages = num_pages; p.block_size = block_size;
  p.block_shift = -1;
  for (int sh = 0; sh < 31; ++sh) if ((1 << sh) == block_size) p.block_shift = sh;
  p.visible_lengths = visible_lengths;
  p.max_len = max_blocks * (int64_t)block_size;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.groups = q_heads / kv_heads;
  p.scaling = scaling;
  return run_dense_decode(p, gate, gate_stride_b, gate_stride_h, out, out_stride_b, out_stride_h, partial_stats,
                          partial_values, chunk_capacity, chunk_tokens, split_counters, batch, head_dim, dtype,
                          (cudaStream_t)stream);
}

extern "C" int anna_gqa_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* key,
                               const void* value, int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t,
                               const int64_t* visible_lengths, const void* gate, int64_t gate_stride_b,
                               int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h,
                               float* partial_stats, float* partial_values, int chunk_capacity, int chunk_tokens,
                               int32_t* split_counters, int batch, int q_heads, int kv_heads, int64_t key_len,
                               int head_dim, float scaling,
                               int dtype, anna_stream_t stream) {
  ANNA_REQUIRE(q && key && value && out, "anna_gqa_decode: null pointer argument");
  ANNA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
               "anna_gqa_decode: query heads (%d) must be a positive multiple of kv heads (%d)", q_heads, kv_heads);
  ANNA_REQUIRE(key_len >= 1, "anna_gqa_decode: key_len must be positive");
  const int vec = dtype == ANNA_DTYPE_F32 ? 4 : 8;
  ANNA_REQUIRE(kv_stride_b % vec == 0 && kv_stride_h % vec == 0 && kv_stride_t % vec == 0,
               "anna_gqa_decode: K/V strides must keep rows 16-byte aligned");
  DenseDecodeParams p{};
  p.q = q; p.q_stride_b = q_stride_b; p.q_stride_h = q_stride_h;
  p.key = key; p.value = value;
  p.page_table = nullptr;
  p.block_size = 1; p.block_shift = 0;
  p.kv_stride_b = kv_stride_b; p.kv_stride_h = kv_stride_h; p.kv_stride_t = kv_stride_t;
  p.visible_lengths = visible_lengths;
  p.max_len = key_len;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.groups = q_heads / kv_heads;
  p.scaling = scaling;
  return run_dense_decode(p, gate, gate_stride_b, gate_stride_h, out, out_stride_b, out_stride_h, partial_stats,
                          partial_values, chunk_capacity, chunk_tokens, split_counters, batch, head_dim, dtype,
                          (cudaStream_t)stream);
}
