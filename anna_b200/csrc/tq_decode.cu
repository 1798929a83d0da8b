// Single-token GQA decode over [packed TurboQuant prefix | un-quantized window ring], CUDA-core path.
//
// Keys are scored straight from their codes in the rotated basis:
//   q . k_hat = norm / D * [ fwht(s1*q) . centroid[idx] + sqrt(pi/2)/sqrt(D) * rnorm * fwht(s2*fwht(s1*q)) . (2*sign-1) ]
// so a CTA rotates its G query heads once (two Walsh-Hadamard passes per head) and never de-quantizes a key into
// the original basis.  Values are de-quantized in registers as code * scale + zero.
#include "decode_core.cuh"
#include "tq_common.cuh"
#include "tq_decode_params.cuh"

#include <cstdlib>

namespace anna {

// Bits of COUNT consecutive coordinates starting at `first` in a row packed with WIDTH bits per coordinate.
template <int COUNT, int WIDTH>
__device__ __forceinline__ uint32_t load_packed_bits(const uint8_t* __restrict__ row, int first) {
  constexpr int kBits = COUNT * WIDTH;
  static_assert(kBits == 4 || kBits == 8 || kBits == 16 || kBits == 32, "unsupported packed width");
  const int bit_off = first * WIDTH;
  const uint8_t* ptr = row + (bit_off >> 3);
  if constexpr (kBits == 32) {
    return __ldg(reinterpret_cast<const uint32_t*>(ptr));
  } else if constexpr (kBits == 16) {
    return __ldg(reinterpret_cast<const uint16_t*>(ptr));
  } else {
    return ((uint32_t)__ldg(ptr) >> (bit_off & 7)) & ((1u << kBits) - 1u);
  }
}

constexpr int kTqUnroll = 2;

template <typename T, int D, int G, int BITS>
__global__ void __launch_bounds__(kDecodeThreads) tq_decode_split_kernel(const TqDecodeParams p) {
  using Cfg = DecodeCfg<T, D, G>;
  constexpr int E = D / 32;
  constexpr int M = BITS - 1;
  constexpr int VS = BITS == 2 ? 2 : 4;
  constexpr int kVec = Cfg::kVec;
  extern __shared__ float smem[];
  __shared__ float sm_cent[1 << M];

  const int chunk = blockIdx.x;
  const int group_tiles = (p.groups + G - 1) / G;
  const int kvh = blockIdx.y / group_tiles;
  const int g0 = (blockIdx.y % group_tiles) * G;
  const int g_count = min(G, p.groups - g0);
  const int b = blockIdx.z;

  int64_t len = p.lengths[b];
  len = max((int64_t)0, min(len, p.max_len));
  if (len == 0) return;
  const int64_t R = p.residual_len;
  const int64_t Lq = len > R ? len - R : 0;
  const int active_window = (int)((len - Lq + p.chunk_tokens - 1) / p.chunk_tokens);
  // slots [0, num_window_chunks) walk the window ring, the others the packed prefix; partials are written so that
  // the active slots of a row stay contiguous: [window chunks | packed chunks]
  int64_t t0, t1;
  int out_slot;
  if (chunk < p.num_window_chunks) {
    if (chunk >= active_window) return;
    t0 = Lq + (int64_t)chunk * p.chunk_tokens;
    t1 = min(len, t0 + p.chunk_tokens);
    out_slot = chunk;
  } else {
    const int packed_chunk = chunk - p.num_window_chunks;
    t0 = (int64_t)packed_chunk * p.chunk_tokens;
    if (t0 >= Lq) return;
    t1 = min(Lq, t0 + p.chunk_tokens);
    out_slot = active_window + packed_chunk;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int sub = lane / Cfg::kLpt;
  const int dl = lane % Cfg::kLpt;
  const int hq0 = kvh * p.groups + g0;

  if (threadIdx.x < (1 << M)) sm_cent[threadIdx.x] = p.centroids[threadIdx.x];

  // ---- rotate the group's queries: q_smem[0] = q, [1] = fwht(s1*q), [2] = fwht(s2*[1]) ---------------------------
  float* q_smem = smem;  // [3][G][D]
  {
    const T* q_ptr = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b;
    for (int g = warp; g < G; g += kDecodeWarps) {
      float w[E];
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const int d = lane * E + j;
        w[j] = g < g_count ? ElemTraits<T>::to_float(q_ptr[(int64_t)(hq0 + g) * p.q_stride_h + d]) : 0.0f;
        q_smem[(0 * G + g) * D + d] = w[j];
        if (p.signs1[d] < 0.0f) w[j] = -w[j];
      }
      warp_fwht<E>(w, lane);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const int d = lane * E + j;
        q_smem[(1 * G + g) * D + d] = w[j];
        if (p.signs2[d] < 0.0f) w[j] = -w[j];
      }
      warp_fwht<E>(w, lane);
#pragma unroll
      for (int j = 0; j < E; ++j) q_smem[(2 * G + g) * D + lane * E + j] = w[j];
    }
  }
  __syncthreads();

  TeamState<T, D, G> st;
  st.reset();

  // ---- packed prefix ---------------------------------------------------------------------------------------------
  const int64_t q_end = min(t1, Lq);
  if (t0 < q_end) {
    const float inv_dim = 1.0f / (float)D;
    const float kappa = 1.2533141373155001f * rsqrtf((float)D);  // sqrt(pi/2) / sqrt(D)
    float q2[G][Cfg::kDpl];
    load_query_from_smem<T, D, G>(st, q_smem + 1 * G * D, dl, p.scaling * inv_dim);
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < Cfg::kDpl; ++i)
        q2[g][i] = q_smem[(2 * G + g) * D + lane_dim<Cfg>(dl, i)] * (p.scaling * inv_dim * kappa);

    const int32_t* table_row = p.block_table + (int64_t)b * p.table_stride;
    constexpr int kStep = kDecodeWarps * Cfg::kTpw * kTqUnroll;
    for (int64_t base = t0 + warp * (Cfg::kTpw * kTqUnroll); base < q_end; base += kStep) {
      float s[kTqUnroll][G];
      float vhat[kTqUnroll][Cfg::kDpl];
      bool valid[kTqUnroll];
#pragma unroll
      for (int u = 0; u < kTqUnroll; ++u) {
        const int64_t t = base + u * Cfg::kTpw + sub;
        valid[u] = false;
        const uint8_t* chunk_ptr = nullptr;
        int tok = 0;
        if (t < q_end) {
          const int32_t pid = table_row[t / p.block_size];
          if (pid >= 0 && pid < p.num_pages) {
            valid[u] = true;
            tok = (int)(t % p.block_size);
            chunk_ptr = p.pages + ((int64_t)pid * p.kv_heads + kvh) * p.layout.chunk_bytes;
          }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) s[u][g] = 0.0f;
#pragma unroll
        for (int i = 0; i < Cfg::kDpl; ++i) vhat[u][i] = 0.0f;
        if (!valid[u]) continue;
        const float norm = __ldg(reinterpret_cast<const float*>(chunk_ptr + p.layout.off_knorm) + tok);
        const float rnorm = __ldg(reinterpret_cast<const float*>(chunk_ptr + p.layout.off_krnorm) + tok);
        const uint8_t* krow = chunk_ptr + p.layout.off_kcodes + tok * p.layout.key_bytes;
        const uint8_t* vrow = chunk_ptr + p.layout.off_vdata + tok * p.layout.value_bytes;
        const T* scales = reinterpret_cast<const T*>(chunk_ptr + p.layout.off_vscale) + tok * p.layout.groups;
        const T* zeros = reinterpret_cast<const T*>(chunk_ptr + p.layout.off_vzero) + tok * p.layout.groups;
#pragma unroll
        for (int c = 0; c < Cfg::kCh; ++c) {
          const int d0 = (c * Cfg::kLpt + dl) * kVec;
          uint32_t idx_bits, sign_bits;  // per coordinate: M index bits, 1 sign bit
          if constexpr (BITS == 3) {
            idx_bits = load_packed_bits<kVec, 2>(krow, d0);
            sign_bits = load_packed_bits<kVec, 1>(krow + D / 4, d0);
          } else {
            idx_bits = load_packed_bits<kVec, BITS>(krow, d0);
            sign_bits = 0;
          }
          float a[G], bsum[G];
#pragma unroll
          for (int g = 0; g < G; ++g) { a[g] = 0.0f; bsum[g] = 0.0f; }
#pragma unroll
          for (int i = 0; i < kVec; ++i) {
            uint32_t code, sbit;
            if constexpr (BITS == 3) {
              code = (idx_bits >> (2 * i)) & 3u;
              sbit = (sign_bits >> i) & 1u;
            } else {
              const uint32_t field = (idx_bits >> (BITS * i)) & ((1u << BITS) - 1u);
              code = field & ((1u << M) - 1u);
              sbit = field >> M;
            }
            const float cv = sm_cent[code];
            const float sv = sbit ? 1.0f : -1.0f;
#pragma unroll
            for (int g = 0; g < G; ++g) {
              a[g] = fmaf(st.q[g][c * kVec + i], cv, a[g]);
              bsum[g] = fmaf(q2[g][c * kVec + i], sv, bsum[g]);
            }
          }
#pragma unroll
          for (int g = 0; g < G; ++g) s[u][g] += norm * fmaf(rnorm, bsum[g], a[g]);

          const uint32_t vbits = load_packed_bits<kVec, VS>(vrow, d0);
          const int grp = d0 / p.value_group;
          const float sc = ElemTraits<T>::to_float(scales[grp]);
          const float zp = ElemTraits<T>::to_float(zeros[grp]);
#pragma unroll
          for (int i = 0; i < kVec; ++i) {
            const float code = (float)((vbits >> (VS * i)) & ((1u << VS) - 1u));
            vhat[u][c * kVec + i] = fmaf(code, sc, zp);
          }
        }
      }
#pragma unroll
      for (int d = Cfg::kLpt / 2; d >= 1; d >>= 1) {
#pragma unroll
        for (int u = 0; u < kTqUnroll; ++u)
#pragma unroll
          for (int g = 0; g < G; ++g) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], d);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float m_new = st.m[g];
#pragma unroll
        for (int u = 0; u < kTqUnroll; ++u) {
          if (!valid[u]) s[u][g] = -INFINITY;
          m_new = fmaxf(m_new, s[u][g]);
        }
        const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
        const float rescale = __expf(st.m[g] - m_safe);
        float lsum = st.l[g] * rescale;
        float pr[kTqUnroll];
#pragma unroll
        for (int u = 0; u < kTqUnroll; ++u) {
          pr[u] = __expf(s[u][g] - m_safe);
          lsum += pr[u];
        }
        st.l[g] = lsum;
        st.m[g] = m_new;
#pragma unroll
        for (int i = 0; i < Cfg::kDpl; ++i) {
          float acc = st.acc[g][i] * rescale;
#pragma unroll
          for (int u = 0; u < kTqUnroll; ++u) acc = fmaf(pr[u], vhat[u][i], acc);
          st.acc[g][i] = acc;
        }
      }
    }
  }

  // ---- un-quantized window ring ------------------------------------------------------------------------------------
  const int64_t w_begin = max(t0, Lq);
  if (w_begin < t1) {
    load_query_from_smem<T, D, G>(st, q_smem, dl, p.scaling);
    const int64_t slot = p.window_slots[b];
    const T* ring_k = reinterpret_cast<const T*>(p.window) + ((slot * 2 + 0) * p.kv_heads + kvh) * R * D;
    const T* ring_v = reinterpret_cast<const T*>(p.window) + ((slot * 2 + 1) * p.kv_heads + kvh) * R * D;
    constexpr int kStep = kDecodeWarps * Cfg::kTpw * kUnroll;
    for (int64_t base = w_begin + warp * (Cfg::kTpw * kUnroll); base < t1; base += kStep) {
      int64_t off[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t t = base + u * Cfg::kTpw + sub;
        off[u] = t < t1 ? (t % R) * D : -1;
      }
      team_consume<T, D, G>(st, ring_k, ring_v, off, dl);
    }
  }
  __syncthreads();  // every warp is done with q_smem before the merge reuses shared memory

  const int64_t part = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity + out_slot;
  cta_merge_store<T, D, G>(st, smem, warp, sub, dl, g_count, p.stats + part * 2, p.values + part * D,
                           (int64_t)p.chunk_capacity * 2, (int64_t)p.chunk_capacity * D);
}

template <typename T, int D, int G, int BITS>
static int launch_tq_split(const TqDecodeParams& p, int batch, cudaStream_t stream) {
  using Cfg = DecodeCfg<T, D, G>;
  const size_t smem_merge = sizeof(float) * (size_t)Cfg::kTeams * G * (D + 2);
  const size_t smem_q = sizeof(float) * (size_t)3 * G * D;
  const size_t smem = smem_merge > smem_q ? smem_merge : smem_q;
  auto kernel = tq_decode_split_kernel<T, D, G, BITS>;
  if (smem > 48 * 1024) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const int group_tiles = (p.groups + G - 1) / G;
  dim3 grid((unsigned)p.num_chunks, (unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
  kernel<<<grid, kDecodeThreads, smem, stream>>>(p);
  return check_launch("tq_decode_split_kernel");
}

}  // namespace anna

using namespace anna;

static int tq_paged_decode_impl(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                const uint8_t* packed_pages, const int32_t* block_table, int64_t table_stride,
                                const void* window, const int64_t* window_slots, const int64_t* lengths,
                                const float* signs1, const float* signs2, const float* centroids,
                                const void* gate, int64_t gate_stride_b, int64_t gate_stride_h, void* out,
                                int64_t out_stride_b, int64_t out_stride_h, float* partial_stats,
                                float* partial_values, int chunk_capacity, int chunk_tokens_in,
                                int32_t* split_counters, void* query_scratch, size_t query_scratch_bytes,
                                int batch, int q_heads, int kv_heads, int head_dim,
                                int block_size, int residual_len, int bits, int value_group, int64_t num_pages,
                                int64_t max_blocks, float scaling, int dtype, void* const* peer_outputs, int num_peers,
                                anna_stream_t stream) {
  ANNA_REQUIRE(num_peers >= 0 && num_peers <= kMaxPeerOutputs && (num_peers == 0 || peer_outputs != nullptr),
               "anna_tq_paged_decode: between 0 and %d peer outputs", kMaxPeerOutputs);
  for (int i = 0; i < num_peers; ++i)
    ANNA_REQUIRE(peer_outputs[i] != nullptr, "anna_tq_paged_decode: null peer output %d", i);
  ANNA_REQUIRE(q && window && window_slots && lengths && signs1 && signs2 && centroids && out,
               "anna_tq_paged_decode: null pointer argument");
  ANNA_REQUIRE(packed_pages != nullptr || num_pages == 0, "anna_tq_paged_decode: null page pool with num_pages > 0");
  ANNA_REQUIRE(block_table != nullptr || max_blocks == 0, "anna_tq_paged_decode: null block table with max_blocks > 0");
  ANNA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
               "anna_tq_paged_decode: query heads (%d) must be a positive multiple of kv heads (%d)", q_heads, kv_heads);
  ANNA_REQUIRE(residual_len >= 1 && block_size >= 1 && max_blocks >= 0, "anna_tq_paged_decode: bad geometry");
  const int vec = dtype == ANNA_DTYPE_F32 ? 4 : 8;
  ANNA_REQUIRE(value_group % vec == 0, "anna_tq_paged_decode: value group %d must be a multiple of %d", value_group, vec);
  TqDecodeParams p{};
  p.q = q; p.q_stride_b = q_stride_b; p.q_stride_h = q_stride_h;
  p.pages = packed_pages; p.block_table = block_table; p.table_stride = table_stride;
  p.window = window; p.window_slots = window_slots; p.lengths = lengths;
  p.signs1 = signs1; p.signs2 = signs2; p.centroids = centroids;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.groups = q_heads / kv_heads;
  p.block_size = block_size; p.residual_len = residual_len; p.value_group = value_group;
  p.block_shift = -1;
  for (int sh = 0; sh < 31; ++sh) if ((1 << sh) == block_size) p.block_shift = sh;
  p.num_pages = num_pages; p.max_blocks = max_blocks;
  p.max_len = max_blocks * (int64_t)block_size + residual_len;
  p.scaling = scaling;
  if (!tq_make_layout(head_dim, bits, block_size, dtype_bytes_of(dtype), value_group, &p.layout))
    return set_error(ANNA_ERR_INVALID, "anna_tq_paged_decode: unsupported geometry D=%d bits=%d S=%d group=%d", head_dim,
                     bits, block_size, value_group);
  int chunk_tokens = 0, num_chunks = 0;
  int rc;
  if (chunk_tokens_in > 0) {
    chunk_tokens = chunk_tokens_in;
    const int64_t nw = (residual_len + chunk_tokens - 1) / chunk_tokens;
    const int64_t nq = (max_blocks * (int64_t)block_size + chunk_tokens - 1) / chunk_tokens;
    num_chunks = (int)(nw + nq);
  } else {
    rc = anna_tq_decode_plan(batch, kv_heads, max_blocks, block_size, residual_len, &chunk_tokens, &num_chunks);
    if (rc != ANNA_OK) return rc;
  }
  if (partial_stats == nullptr || partial_values == nullptr)
    return set_error(ANNA_ERR_WORKSPACE, "anna_tq_paged_decode needs partial_stats and partial_values scratch buffers");
  if (num_chunks > chunk_capacity)
    return set_error(ANNA_ERR_WORKSPACE, "split-K scratch holds %d chunks per head, %d needed", chunk_capacity, num_chunks);
  SplitWorkspace ws{partial_stats, partial_values, chunk_capacity};
  p.stats = ws.stats; p.values = ws.values;
  p.chunk_tokens = chunk_tokens; p.num_chunks = num_chunks; p.chunk_capacity = chunk_capacity;
  p.num_window_chunks = (residual_len + chunk_tokens - 1) / chunk_tokens;
  {
    const size_t need = tq_query_scratch_bytes(batch, q_heads, kv_heads, head_dim);
    const bool fits = query_scratch != nullptr && query_scratch_bytes >= need &&
                      (reinterpret_cast<uintptr_t>(query_scratch) & 15u) == 0;
    p.query_frags = fits ? query_scratch : nullptr;
  }
  if (tq_split_mma_applicable(p, head_dim, dtype)) {
    const bool umma = tq_split_umma_applicable(p, head_dim, bits, dtype);
    if (split_counters != nullptr && num_chunks <= kFusedMaxChunks) {
      p.fused = FusedCombine{split_counters, out, out_stride_b, out_stride_h, gate, gate_stride_b, gate_stride_h};
      for (int i = 0; i < num_peers; ++i) p.fused.peers[i] = peer_outputs[i];
      p.fused.num_peers = num_peers;
      return umma ? launch_tq_split_umma(p, batch, bits, dtype, (cudaStream_t)stream)
                  : launch_tq_split_mma(p, batch, head_dim, bits, dtype, (cudaStream_t)stream);
    }
    if (num_peers > 0)
      return set_error(ANNA_ERR_UNSUPPORTED, "peer outputs need the fused merge (split counters, at most %d chunks)",
                       kFusedMaxChunks);
    rc = umma ? launch_tq_split_umma(p, batch, bits, dtype, (cudaStream_t)stream)
              : launch_tq_split_mma(p, batch, head_dim, bits, dtype, (cudaStream_t)stream);
    if (rc != ANNA_OK) return rc;
    return launch_split_combine(ws, nullptr, p.lengths, -1, p.max_len, residual_len, gate, gate_stride_b, gate_stride_h,
                                out, out_stride_b, out_stride_h, batch, q_heads, head_dim, chunk_tokens, num_chunks,
                                dtype, (cudaStream_t)stream);
  }
  if (num_peers > 0)
    return set_error(ANNA_ERR_UNSUPPORTED, "peer outputs need the tensor-core decode path (16-bit cache, head_dim 128/256)");
  const int gpad = padded_group(p.groups);
  rc = ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    return ANNA_DISPATCH_TQ_DIM(head_dim, D, [&]() -> int {
      return ANNA_DISPATCH_GROUP(gpad, G, [&]() -> int {
        return ANNA_DISPATCH_TQ_BITS(bits, BITS, [&]() -> int {
          return launch_tq_split<T, D, G, BITS>(p, batch, (cudaStream_t)stream);
        });
      });
    });
  });
  if (rc != ANNA_OK) return rc;
  return launch_split_combine(ws, nullptr, p.lengths, -1, p.max_len, residual_len, gate, gate_stride_b, gate_stride_h,
                              out, out_stride_b, out_stride_h, batch, q_heads, head_dim, chunk_tokens, num_chunks,
                              dtype, (cudaStream_t)stream);
}

extern "C" int anna_tq_paged_decode(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                    const uint8_t* packed_pages, const int32_t* block_table, int64_t table_stride,
                                    const void* window, const int64_t* window_slots, const int64_t* lengths,
                                    const float* signs1, const float* signs2, const float* centroids,
                                    const void* gate, int64_t gate_stride_b, int64_t gate_stride_h, void* out,
                                    int64_t out_stride_b, int64_t out_stride_h, float* partial_stats,
                                    float* partial_values, int chunk_capacity, int chunk_tokens_in,
                                    int32_t* split_counters, void* query_scratch, size_t query_scratch_bytes,
                                    int batch, int q_heads, int kv_heads, int head_dim,
                                    int block_size, int residual_len, int bits, int value_group, int64_t num_pages,
                                    int64_t max_blocks, float scaling, int dtype, anna_stream_t stream) {
  return tq_paged_decode_impl(q, q_stride_b, q_stride_h, packed_pages, block_table, table_stride, window, window_slots,
                              lengths, signs1, signs2, centroids, gate, gate_stride_b, gate_stride_h, out, out_stride_b,
                              out_stride_h, partial_stats, partial_values, chunk_capacity, chunk_tokens_in,
                              split_counters, query_scratch, query_scratch_bytes, batch, q_heads, kv_heads, head_dim,
                              block_size, residual_len, bits, value_group, num_pages, max_blocks, scaling, dtype,
                              nullptr, 0, stream);
}

extern "C" int anna_tq_paged_decode_peers(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                          const uint8_t* packed_pages, const int32_t* block_table,
                                          int64_t table_stride, const void* window, const int64_t* window_slots,
                                          const int64_t* lengths, const float* signs1, const float* signs2,
                                          const float* centroids, const void* gate, int64_t gate_stride_b,
                                          int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h,
                                          float* partial_stats, float* partial_values, int chunk_capacity,
                                          int chunk_tokens_in, int32_t* split_counters, void* query_scratch,
                                          size_t query_scratch_bytes, int batch, int q_heads, int kv_heads,
                                          int head_dim, int block_size, int residual_len, int bits, int value_group,
                                          int64_t num_pages, int64_t max_blocks, float scaling, int dtype,
                                          void* const* peer_outputs, int num_peers, anna_stream_t stream) {
  return tq_paged_decode_impl(q, q_stride_b, q_stride_h, packed_pages, block_table, table_stride, window, window_slots,
                              lengths, signs1, signs2, centroids, gate, gate_stride_b, gate_stride_h, out, out_stride_b,
                              out_stride_h, partial_stats, partial_values, chunk_capacity, chunk_tokens_in,
                              split_counters, query_scratch, query_scratch_bytes, batch, q_heads, kv_heads, head_dim,
                              block_size, residual_len, bits, value_group, num_pages, max_blocks, scaling, dtype,
                              peer_outputs, num_peers, stream);
}

extern "C" size_t anna_tq_query_scratch_bytes(int batch, int q_heads, int kv_heads, int head_dim) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || q_heads % kv_heads != 0) return 0;
  return tq_query_scratch_bytes(batch, q_heads, kv_heads, head_dim);
}

extern "C" int anna_tq_decode_plan(int batch, int kv_heads, int64_t max_blocks, int block_size, int residual_len,
                                   int* chunk_tokens, int* num_chunks) {
  ANNA_REQUIRE(max_blocks >= 0 && block_size >= 1 && residual_len >= 1, "anna_tq_decode_plan: bad geometry");
  ANNA_REQUIRE(batch > 0 && kv_heads > 0, "anna_tq_decode_plan: batch and kv_heads must be positive");
  ANNA_REQUIRE(chunk_tokens != nullptr && num_chunks != nullptr, "anna_tq_decode_plan: null output pointer");
  const int64_t max_q = max_blocks * (int64_t)block_size;
  // Packed tokens are 3-6x smaller than 16-bit ones and every CTA pays a fixed fragment-load / merge cost, so the
  // chunks are longer than for the un-quantized path: the largest of 4096 ... 64 tokens that still gives ~8 CTAs per SM
  // (measured: 64 x 32768-token rows run 4.5 % faster with 4096-token chunks than with 1024-token ones, and every
  // problem that is short of CTAs gets slower when the chunks shrink further).
  const int64_t streams = (int64_t)batch * kv_heads;
  int64_t ct = 4096;
  while (ct > 64 && streams * ((max_q + residual_len + ct - 1) / ct) < 148 * 8) ct >>= 1;
  *chunk_tokens = (int)ct;
  *num_chunks = (int)((residual_len + ct - 1) / ct + (max_q + ct - 1) / ct);
  return ANNA_OK;
}
