// Single-token GQA decode over (dense de-quantized keys | packed values | un-quantized residual): the operand set of
// torch.ops.anna.gqa_decode_splitkv_turboquant_fused_out.  CUDA-core path built from the same team machinery as the
// dense split kernel; values are de-quantized in registers as code * scale + zero.
#include "decode_core.cuh"

namespace anna {

struct TqValuesParams {
  const void* q;
  int64_t q_stride_b, q_stride_h;
  const void* quantized_key;
  int64_t qk_stride_b, qk_stride_h, qk_stride_t;
  const uint8_t* value_data;
  int64_t vd_stride_b, vd_stride_h, vd_stride_t;
  const void* value_scales;
  const void* value_zeros;
  int64_t vs_stride_b, vs_stride_h, vs_stride_t;
  const void* residual_key;
  const void* residual_value;
  int64_t r_stride_b, r_stride_h, r_stride_t;
  float* stats;
  float* values;
  int q_heads, kv_heads, groups;
  int64_t quantized_len, residual_len;
  int value_bits, value_group;
  int chunk_tokens, num_chunks, chunk_capacity;
  float scaling;
};

template <typename T, int D, int G>
__global__ void __launch_bounds__(kDecodeThreads) tq_values_decode_split_kernel(const TqValuesParams p) {
  using Cfg = DecodeCfg<T, D, G>;
  constexpr int kVec = Cfg::kVec;
  extern __shared__ float smem[];
  const int chunk = blockIdx.x;
  const int group_tiles = (p.groups + G - 1) / G;
  const int kvh = blockIdx.y / group_tiles;
  const int g0 = (blockIdx.y % group_tiles) * G;
  const int g_count = min(G, p.groups - g0);
  const int b = blockIdx.z;
  const int64_t len = p.quantized_len + p.residual_len;
  const int64_t t0 = (int64_t)chunk * p.chunk_tokens;
  if (t0 >= len) return;
  const int64_t t1 = min(len, t0 + p.chunk_tokens);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int sub = lane / Cfg::kLpt;
  const int dl = lane % Cfg::kLpt;
  const int hq0 = kvh * p.groups + g0;

  float* q_smem = smem;
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
  __syncthreads();

  const T* qk = reinterpret_cast<const T*>(p.quantized_key) + (int64_t)b * p.qk_stride_b + (int64_t)kvh * p.qk_stride_h;
  const uint8_t* vd = p.value_data + (int64_t)b * p.vd_stride_b + (int64_t)kvh * p.vd_stride_h;
  const T* vs = reinterpret_cast<const T*>(p.value_scales) + (int64_t)b * p.vs_stride_b + (int64_t)kvh * p.vs_stride_h;
  const T* vz = reinterpret_cast<const T*>(p.value_zeros) + (int64_t)b * p.vs_stride_b + (int64_t)kvh * p.vs_stride_h;
  const T* rk = reinterpret_cast<const T*>(p.residual_key) + (int64_t)b * p.r_stride_b + (int64_t)kvh * p.r_stride_h;
  const T* rv = reinterpret_cast<const T*>(p.residual_value) + (int64_t)b * p.r_stride_b + (int64_t)kvh * p.r_stride_h;
  const int storage = p.value_bits == 2 ? 2 : 4;
  const uint32_t code_mask = (1u << storage) - 1u;

  // ---- quantized prefix: dense keys, packed values -------------------------------------------------------------------
  const int64_t q_end = min(t1, p.quantized_len);
  constexpr int kStepQ = kDecodeWarps * Cfg::kTpw;
  for (int64_t base = t0 + warp * Cfg::kTpw; base < q_end; base += kStepQ) {
    const int64_t t = base + sub;
    const bool ok = t < q_end;
    float s[G];
    float vf[Cfg::kDpl];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.0f;
#pragma unroll
    for (int c = 0; c < Cfg::kCh; ++c) {
      const int d0 = (c * Cfg::kLpt + dl) * kVec;
      float kf[kVec];
      if (ok) {
        widen16<T>(ldg_stream16(qk + t * p.qk_stride_t + d0), kf);
      } else {
#pragma unroll
        for (int i = 0; i < kVec; ++i) kf[i] = 0.0f;
      }
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < kVec; ++i) s[g] = fmaf(st.q[g][c * kVec + i], kf[i], s[g]);
      float sc = 0.0f, zp = 0.0f;
      uint32_t bits = 0;
      if (ok) {
        const int grp = d0 / p.value_group;
        sc = ElemTraits<T>::to_float(vs[t * p.vs_stride_t + grp]);
        zp = ElemTraits<T>::to_float(vz[t * p.vs_stride_t + grp]);
        const uint8_t* src = vd + t * p.vd_stride_t + (d0 * storage) / 8;
        const int nbytes = kVec * storage / 8;  // 1, 2 or 4
        for (int k = 0; k < nbytes; ++k) bits |= (uint32_t)__ldg(src + k) << (8 * k);
      }
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const float code = (float)((bits >> (storage * i)) & code_mask);
        vf[c * kVec + i] = ok ? fmaf(code, sc, zp) : 0.0f;
      }
    }
#pragma unroll
    for (int d = Cfg::kLpt / 2; d >= 1; d >>= 1)
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] += __shfl_xor_sync(0xffffffffu, s[g], d);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float score = ok ? s[g] : -INFINITY;
      const float m_new = fmaxf(st.m[g], score);
      const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
      const float rescale = __expf(st.m[g] - m_safe);
      const float pr = __expf(score - m_safe);
      st.l[g] = st.l[g] * rescale + pr;
      st.m[g] = m_new;
#pragma unroll
      for (int i = 0; i < Cfg::kDpl; ++i) st.acc[g][i] = fmaf(pr, vf[i], st.acc[g][i] * rescale);
    }
  }

  // ---- residual tokens: dense keys and values -------------------------------------------------------------------------
  const int64_t r_begin = max(t0, p.quantized_len);
  if (r_begin < t1) {
    constexpr int kStep = kDecodeWarps * Cfg::kTpw * kUnroll;
    for (int64_t base = r_begin + warp * (Cfg::kTpw * kUnroll); base < t1; base += kStep) {
      int64_t off[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t t = base + u * Cfg::kTpw + sub;
        off[u] = t < t1 ? (t - p.quantized_len) * p.r_stride_t : -1;
      }
      team_consume<T, D, G>(st, rk, rv, off, dl);
    }
  }
  const int64_t part = ((int64_t)b * p.q_heads + hq0) * p.chunk_capacity + chunk;
  cta_merge_store<T, D, G>(st, smem, warp, sub, dl, g_count, p.stats + part * 2, p.values + part * D,
                           (int64_t)p.chunk_capacity * 2, (int64_t)p.chunk_capacity * D);
}

template <typename T, int D, int G>
static int launch_tq_values(const TqValuesParams& p, int batch, cudaStream_t stream) {
  using Cfg = DecodeCfg<T, D, G>;
  const size_t smem_merge = sizeof(float) * (size_t)Cfg::kTeams * G * (D + 2);
  const size_t smem_q = sizeof(float) * (size_t)G * D;
  const size_t smem = smem_merge > smem_q ? smem_merge : smem_q;
  auto kernel = tq_values_decode_split_kernel<T, D, G>;
  if (smem > 48 * 1024) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const int group_tiles = (p.groups + G - 1) / G;
  dim3 grid((unsigned)p.num_chunks, (unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
  kernel<<<grid, kDecodeThreads, smem, stream>>>(p);
  return check_launch("tq_values_decode_split_kernel");
}

}  // namespace anna

using namespace anna;

extern "C" int anna_gqa_decode_turboquant_values(
    const void* q, int64_t q_stride_b, int64_t q_stride_h, const void* quantized_key, int64_t qk_stride_b,
    int64_t qk_stride_h, int64_t qk_stride_t, const uint8_t* value_data, int64_t vd_stride_b, int64_t vd_stride_h,
    int64_t vd_stride_t, const void* value_scales, const void* value_zeros, int64_t vs_stride_b, int64_t vs_stride_h,
    int64_t vs_stride_t, const void* residual_key, const void* residual_value, int64_t r_stride_b, int64_t r_stride_h,
    int64_t r_stride_t, const void* gate, int64_t gate_stride_b, int64_t gate_stride_h, void* out, int64_t out_stride_b,
    int64_t out_stride_h, float* partial_stats, float* partial_values, int chunk_capacity, int chunk_tokens, int batch,
    int q_heads, int kv_heads, int64_t quantized_len, int64_t residual_len, int head_dim, int value_bits,
    int value_group, float scaling, int dtype, anna_stream_t stream) {
  ANNA_REQUIRE(q && quantized_key && value_data && value_scales && value_zeros && out,
               "anna_gqa_decode_turboquant_values: null pointer argument");
  ANNA_REQUIRE(residual_len == 0 || (residual_key && residual_value),
               "anna_gqa_decode_turboquant_values: residual tensors are required when residual_len > 0");
  ANNA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
               "anna_gqa_decode_turboquant_values: query heads (%d) must be a positive multiple of kv heads (%d)",
               q_heads, kv_heads);
  ANNA_REQUIRE(quantized_len >= 1 && residual_len >= 0, "anna_gqa_decode_turboquant_values: quantized_len must be >= 1");
  ANNA_REQUIRE(value_bits >= 2 && value_bits <= 4, "TurboQuant value_bits must be 2, 3, or 4");
  const int vec = dtype == ANNA_DTYPE_F32 ? 4 : 8;
  ANNA_REQUIRE(value_group > 0 && head_dim % value_group == 0 && value_group % vec == 0,
               "anna_gqa_decode_turboquant_values: value_group %d must divide head_dim %d and be a multiple of %d",
               value_group, head_dim, vec);
  ANNA_REQUIRE(qk_stride_b % vec == 0 && qk_stride_h % vec == 0 && qk_stride_t % vec == 0 && r_stride_b % vec == 0 &&
                   r_stride_h % vec == 0 && r_stride_t % vec == 0,
               "anna_gqa_decode_turboquant_values: key strides must keep rows 16-byte aligned");
  TqValuesParams p{};
  p.q = q; p.q_stride_b = q_stride_b; p.q_stride_h = q_stride_h;
  p.quantized_key = quantized_key; p.qk_stride_b = qk_stride_b; p.qk_stride_h = qk_stride_h; p.qk_stride_t = qk_stride_t;
  p.value_data = value_data; p.vd_stride_b = vd_stride_b; p.vd_stride_h = vd_stride_h; p.vd_stride_t = vd_stride_t;
  p.value_scales = value_scales; p.value_zeros = value_zeros;
  p.vs_stride_b = vs_stride_b; p.vs_stride_h = vs_stride_h; p.vs_stride_t = vs_stride_t;
  p.residual_key = residual_key ? residual_key : quantized_key;
  p.residual_value = residual_value ? residual_value : quantized_key;
  p.r_stride_b = r_stride_b; p.r_stride_h = r_stride_h; p.r_stride_t = r_stride_t;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.groups = q_heads / kv_heads;
  p.quantized_len = quantized_len; p.residual_len = residual_len;
  p.value_bits = value_bits; p.value_group = value_group;
  p.scaling = scaling;
  const int64_t key_len = quantized_len + residual_len;
  int ct = 0, chunks = 0;
  int rc = resolve_split(batch, kv_heads, key_len, chunk_tokens, chunk_capacity, partial_stats, partial_values, &ct,
                         &chunks);
  if (rc != ANNA_OK) return rc;
  SplitWorkspace ws{partial_stats, partial_values, chunk_capacity};
  p.stats = ws.stats; p.values = ws.values;
  p.chunk_tokens = ct; p.num_chunks = chunks; p.chunk_capacity = chunk_capacity;
  const int gpad = padded_group(p.groups);
  rc = ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    return ANNA_DISPATCH_DIM(head_dim, D, [&]() -> int {
      return ANNA_DISPATCH_GROUP(gpad, G, [&]() -> int {
        return launch_tq_values<T, D, G>(p, batch, (cudaStream_t)stream);
      });
    });
  });
  if (rc != ANNA_OK) return rc;
  return launch_split_combine(ws, nullptr, nullptr, key_len, key_len, 0, gate, gate_stride_b, gate_stride_h, out,
                              out_stride_b, out_stride_h, batch, q_heads, head_dim, ct, chunks, dtype,
                              (cudaStream_t)stream);
}
