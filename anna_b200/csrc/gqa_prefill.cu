// Multi-token (prefill / chunked-prefill) grouped-query attention over dense K/V, tensor cores, 16-bit dtypes.
//
// Semantics of grouped_query_attention (src/anna/model/ops.py:1552-1574) for the masks the model builds
// (ops.py:1840-1852, :2008-2016): row r sees its first key_lengths[r] keys (visible_mask / key_padding_mask in prefix
// form); with the causal flag, query t of the chunk sits at position key_lengths[r] - T + t and sees keys up to and
// including its own position.  softmax in fp32, output in the query dtype, rows without any visible key give zeros.
//
// A CTA (4 warps) owns 128 query rows of one query head, a warp two 16-row tiles of them (64 rows and one tile per
// warp at head_dim 256), so every K / V fragment read from shared memory feeds four MMAs.  Per 32-key tile:
//   K / V tile --cp.async (2 stages, zero-filled past the row's keys)--> xor-swizzled shared memory
//   S[16 x 32]  = Q . K^T          Q fragments by ldmatrix from the staged query tile, K by ldmatrix (4 n-tiles x D/16)
//   mask, online softmax in fp32 on the C fragments (row reductions over the 4 lanes of a quad)
//   O[16 x D]  += P . V            P re-packed from the C fragments (no shuffle), V by ldmatrix.trans
// Key tiles above the causal diagonal of the CTA's last query row are never loaded.
#include "mma_utils.cuh"
#include "prefill_params.cuh"

namespace anna {

// mma.sync m16n8k16 without the volatile qualifier (a pure function of its operands): the compiler may then move the
// independent accumulations around the fragment loads, whose order is fixed by hand below.
template <typename T>
__device__ __forceinline__ void mma_pure(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_pure<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_pure<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int kPrefillWarps = 4;
constexpr int kPrefillThreads = kPrefillWarps * 32;

#ifndef ANNA_PREFILL_MT
#define ANNA_PREFILL_MT 2
#endif
template <int D>
struct PrefillCfg {
  // 16-row query tiles per warp: with two, every K / V fragment loaded from shared memory feeds four MMAs instead of two
  static constexpr int kMT = D <= 128 ? ANNA_PREFILL_MT : 1;
  static constexpr int kRows = kPrefillWarps * 16 * kMT;  // query rows per CTA
  static constexpr int kKeys = (D >= 256 || kMT > 1) ? 32 : 64;  // keys per tile (bounded by the score registers)
  static constexpr int kRowBytes = D * 2;
  static constexpr int kChunks = D / 8;                  // 16-byte chunks per row
  static constexpr int kQBytes = kRows * kRowBytes;
#ifndef ANNA_PREFILL_SUBS
#define ANNA_PREFILL_SUBS 1
#endif
  // a stage may hold kSubs key tiles (one CTA barrier pair per kStageKeys keys); two measured the same as one
  static constexpr int kSubs = D <= 128 ? ANNA_PREFILL_SUBS : 1;
  static constexpr int kStageKeys = kKeys * kSubs;
  static constexpr int kTileBytes = kStageKeys * kRowBytes;
  static constexpr int kSmemBytes = kQBytes + 4 * kTileBytes;  // Q | K0 K1 | V0 V1
  static constexpr int kSteps = D / 16;
  static constexpr int kNTiles = kKeys / 8;
};

// rows [row0, row0 + rows) of a [*, D] matrix with token stride `stride` -> swizzled tile; rows >= limit are zero-filled
template <typename T, int D>
__device__ __forceinline__ void prefill_load_tile(uint32_t dst, const T* base, int64_t stride, int64_t row0, int rows,
                                                  int64_t limit) {
  constexpr int kChunks = D / 8;
  for (int item = threadIdx.x; item < rows * kChunks; item += kPrefillThreads) {
    const int r = item / kChunks;
    const int c = item % kChunks;
    const bool ok = row0 + r < limit;
    const T* src = base + (ok ? (row0 + r) * stride + c * 8 : 0);
    cp_async16(dst + swizzled_offset(r, c, D * 2), src, ok ? 16 : 0);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kPrefillThreads, 2) gqa_prefill_mma_kernel(const PrefillParams p) {
  using Cfg = PrefillCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int MT = Cfg::kMT;
  // the query tiles with the most visible keys (the last ones of a causal chunk) are scheduled first
#ifndef ANNA_PREFILL_HEAVY_FIRST
#define ANNA_PREFILL_HEAVY_FIRST 1
#endif
  const int m0 = (ANNA_PREFILL_HEAVY_FIRST ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x) * Cfg::kRows;
  const int hq = blockIdx.y;
  const int b = blockIdx.z;
  const int kvh = hq / p.groups;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int gid = lane >> 2;
  const int tig = lane & 3;
  const int mi = lane >> 3;  // ldmatrix: lanes 8i .. 8i+7 give the row addresses of matrix i
  const int l8 = lane & 7;

  int64_t n_keys = p.key_lengths != nullptr ? p.key_lengths[b] : p.key_len;
  n_keys = max((int64_t)0, min(n_keys, p.key_len));
  const int64_t past = n_keys - p.q_len;  // position of the chunk's first query (negative: the row is shorter than the chunk)
  const int last_row = min(m0 + Cfg::kRows, p.q_len) - 1;
  int64_t cta_limit = p.causal ? min(n_keys, past + last_row + 1) : n_keys;
  cta_limit = max(cta_limit, (int64_t)0);
  const int n_tiles = (int)((cta_limit + Cfg::kStageKeys - 1) / Cfg::kStageKeys);

  const T* q_base = reinterpret_cast<const T*>(p.q) + b * p.q_stride_b + hq * p.q_stride_h;
  const T* k_base = reinterpret_cast<const T*>(p.k) + b * p.kv_stride_b + kvh * p.kv_stride_h;
  const T* v_base = reinterpret_cast<const T*>(p.v) + b * p.kv_stride_b + kvh * p.kv_stride_h;
  const uint32_t q_s = smem_u32(smem_raw);
  const uint32_t k_s = q_s + Cfg::kQBytes;
  const uint32_t v_s = k_s + 2 * Cfg::kTileBytes;

  prefill_load_tile<T, D>(q_s, q_base, p.q_stride_t, m0, Cfg::kRows, p.q_len);
  if (n_tiles > 0) {
    prefill_load_tile<T, D>(k_s, k_base, p.kv_stride_t, 0, Cfg::kStageKeys, n_keys);
    prefill_load_tile<T, D>(v_s, v_base, p.kv_stride_t, 0, Cfg::kStageKeys, n_keys);
  }
  cp_async_commit();

  // rows gid and gid + 8 of the warp's MT query tiles
  int row[MT][2];
  int64_t lim[MT][2];
  float m_run[MT][2], l_run[MT][2];
  float o[MT][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      row[mt][h] = m0 + (warp * MT + mt) * 16 + gid + 8 * h;
      lim[mt][h] = p.causal ? min(n_keys, past + row[mt][h] + 1) : n_keys;
      m_run[mt][h] = -INFINITY;
      l_run[mt][h] = 0.0f;
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) o[mt][j][r] = 0.0f;
  }

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_tiles) {
      const int64_t key0 = (int64_t)(it + 1) * Cfg::kStageKeys;
      prefill_load_tile<T, D>(k_s + (stage ^ 1) * Cfg::kTileBytes, k_base, p.kv_stride_t, key0, Cfg::kStageKeys, n_keys);
      prefill_load_tile<T, D>(v_s + (stage ^ 1) * Cfg::kTileBytes, v_base, p.kv_stride_t, key0, Cfg::kStageKeys, n_keys);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    for (int sub = 0; sub < Cfg::kSubs; ++sub) {
    const int64_t sub_key0 = (int64_t)it * Cfg::kStageKeys + sub * Cfg::kKeys;
    if (sub_key0 >= cta_limit) break;  // nothing visible to any row of the CTA (uniform)
    const uint32_t k_tile = k_s + stage * Cfg::kTileBytes + sub * Cfg::kKeys * Cfg::kRowBytes;
    const uint32_t v_tile = v_s + stage * Cfg::kTileBytes + sub * Cfg::kKeys * Cfg::kRowBytes;

    // ---- S = Q . K^T ---------------------------------------------------------------------------------------------------
    float s[MT][Cfg::kNTiles][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < Cfg::kNTiles; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) s[mt][j][r] = 0.0f;
    {
      // fragment loads run one item ahead of the MMAs that consume them (item = one k-step of one pair of n-tiles)
      constexpr int kPairs = Cfg::kNTiles / 2;
      constexpr int kItems = Cfg::kSteps * kPairs;
      uint32_t a[2][MT][4], bk[2][4];
      auto load_a = [&](int ks, uint32_t (&dst)[MT][4]) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          ldmatrix_x4(dst[mt], q_s + swizzled_offset((warp * MT + mt) * 16 + (mi & 1) * 8 + l8, 2 * ks + (mi >> 1),
                                                     Cfg::kRowBytes));
      };
      auto load_b = [&](int ks, int jp, uint32_t (&dst)[4]) {
        ldmatrix_x4(dst, k_tile + swizzled_offset(jp * 16 + (mi >> 1) * 8 + l8, 2 * ks + (mi & 1), Cfg::kRowBytes));
      };
      load_a(0, a[0]);
      load_b(0, 0, bk[0]);
#pragma unroll
      for (int item = 0; item < kItems; ++item) {
        const int ks = item / kPairs, jp = item % kPairs;
        if (item + 1 < kItems) {
          const int ks1 = (item + 1) / kPairs, jp1 = (item + 1) % kPairs;
          if (jp1 == 0) load_a(ks1, a[ks1 & 1]);
          load_b(ks1, jp1, bk[(item + 1) & 1]);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_pure<T>(s[mt][2 * jp], a[ks & 1][mt], bk[item & 1][0], bk[item & 1][1]);
          mma_pure<T>(s[mt][2 * jp + 1], a[ks & 1][mt], bk[item & 1][2], bk[item & 1][3]);
        }
      }
    }

    // ---- mask + online softmax (log2 units) -----------------------------------------------------------------------------
    const int64_t key_base = sub_key0 + 2 * tig;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < Cfg::kNTiles; ++j) {
        const int64_t key = key_base + 8 * j;
        s[mt][j][0] = key < lim[mt][0] ? s[mt][j][0] * p.scale_log2 : -INFINITY;
        s[mt][j][1] = key + 1 < lim[mt][0] ? s[mt][j][1] * p.scale_log2 : -INFINITY;
        s[mt][j][2] = key < lim[mt][1] ? s[mt][j][2] * p.scale_log2 : -INFINITY;
        s[mt][j][3] = key + 1 < lim[mt][1] ? s[mt][j][3] * p.scale_log2 : -INFINITY;
        mx[0] = fmaxf(mx[0], fmaxf(s[mt][j][0], s[mt][j][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[mt][j][2], s[mt][j][3]));
      }
#pragma unroll
      for (int d = 1; d <= 2; d <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], d));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], d));
      }
      float alpha[2], m_safe[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float m_new = fmaxf(m_run[mt][r], mx[r]);
        m_safe[r] = m_new == -INFINITY ? 0.0f : m_new;
        alpha[r] = ex2_fast(m_run[mt][r] - m_safe[r]);  // 0 on the first visible tile (m_run = -inf)
        m_run[mt][r] = m_new;
        l_run[mt][r] *= alpha[r];
      }
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        o[mt][j][0] *= alpha[0];
        o[mt][j][1] *= alpha[0];
        o[mt][j][2] *= alpha[1];
        o[mt][j][3] *= alpha[1];
      }
#pragma unroll
      for (int j = 0; j < Cfg::kNTiles; ++j) {
        s[mt][j][0] = ex2_fast(s[mt][j][0] - m_safe[0]);
        s[mt][j][1] = ex2_fast(s[mt][j][1] - m_safe[0]);
        s[mt][j][2] = ex2_fast(s[mt][j][2] - m_safe[1]);
        s[mt][j][3] = ex2_fast(s[mt][j][3] - m_safe[1]);
        l_run[mt][0] += s[mt][j][0] + s[mt][j][1];
        l_run[mt][1] += s[mt][j][2] + s[mt][j][3];
      }
    }

    // ---- O += P . V ------------------------------------------------------------------------------------------------------
    {
      constexpr int kDPairs = D / 16;
      constexpr int kItems = (Cfg::kKeys / 16) * kDPairs;
      uint32_t bv[2][4];
      auto load_v = [&](int kk, int dp, uint32_t (&dst)[4]) {
        ldmatrix_x4_trans(dst, v_tile + swizzled_offset(kk * 16 + (mi & 1) * 8 + l8, 2 * dp + (mi >> 1), Cfg::kRowBytes));
      };
      // P as A fragments: the C fragments of two neighbouring n-tiles are exactly the A fragment of one k-step
      uint32_t pa[MT][Cfg::kKeys / 16][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int kk = 0; kk < Cfg::kKeys / 16; ++kk) {
          pa[mt][kk][0] = pack2<T>(s[mt][2 * kk][0], s[mt][2 * kk][1]);
          pa[mt][kk][1] = pack2<T>(s[mt][2 * kk][2], s[mt][2 * kk][3]);
          pa[mt][kk][2] = pack2<T>(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
          pa[mt][kk][3] = pack2<T>(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
        }
      load_v(0, 0, bv[0]);
#pragma unroll
      for (int item = 0; item < kItems; ++item) {
        const int kk = item / kDPairs, dp = item % kDPairs;
        if (item + 1 < kItems) load_v((item + 1) / kDPairs, (item + 1) % kDPairs, bv[(item + 1) & 1]);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_pure<T>(o[mt][2 * dp], pa[mt][kk], bv[item & 1][0], bv[item & 1][1]);
          mma_pure<T>(o[mt][2 * dp + 1], pa[mt][kk], bv[item & 1][2], bv[item & 1][3]);
        }
      }
    }
    }  // sub
    __syncthreads();  // the stage is refilled by the next iteration's loads
  }
  cp_async_wait<0>();

  // ---- normalise and store -------------------------------------------------------------------------------------------------
  T* out_base = reinterpret_cast<T*>(p.out) + b * p.out_stride_b + hq * p.out_stride_h;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int d = 1; d <= 2; d <<= 1) {
      l_run[mt][0] += __shfl_xor_sync(0xffffffffu, l_run[mt][0], d);
      l_run[mt][1] += __shfl_xor_sync(0xffffffffu, l_run[mt][1], d);
    }
    const float inv_lo = l_run[mt][0] > 0.0f ? 1.0f / l_run[mt][0] : 0.0f;
    const float inv_hi = l_run[mt][1] > 0.0f ? 1.0f / l_run[mt][1] : 0.0f;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int col = 8 * j + 2 * tig;
      if (row[mt][0] < p.q_len)
        *reinterpret_cast<uint32_t*>(out_base + row[mt][0] * p.out_stride_t + col) =
            pack2<T>(o[mt][j][0] * inv_lo, o[mt][j][1] * inv_lo);
      if (row[mt][1] < p.q_len)
        *reinterpret_cast<uint32_t*>(out_base + row[mt][1] * p.out_stride_t + col) =
            pack2<T>(o[mt][j][2] * inv_hi, o[mt][j][3] * inv_hi);
    }
  }
}

template <typename T, int D>
static int launch_prefill(const PrefillParams& p, int batch, int q_heads, cudaStream_t stream) {
  using Cfg = PrefillCfg<D>;
  auto kernel = gqa_prefill_mma_kernel<T, D>;
  static bool configured[64] = {};
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !configured[device]) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  dim3 grid((unsigned)((p.q_len + Cfg::kRows - 1) / Cfg::kRows), (unsigned)q_heads, (unsigned)batch);
  kernel<<<grid, kPrefillThreads, Cfg::kSmemBytes, stream>>>(p);
  return check_launch("gqa_prefill_mma_kernel");
}

}  // namespace anna

using namespace anna;

extern "C" int anna_gqa_prefill(const void* q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                                const void* key, const void* value, int64_t kv_stride_b, int64_t kv_stride_h,
                                int64_t kv_stride_t, const int64_t* key_lengths, void* out, int64_t out_stride_b,
                                int64_t out_stride_h, int64_t out_stride_t, int batch, int q_heads, int kv_heads,
                                int q_len, int64_t key_len, int head_dim, float scaling, int causal, int dtype,
                                anna_stream_t stream) {
  ANNA_REQUIRE(q && key && value && out, "anna_gqa_prefill: null pointer argument");
  ANNA_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
               "anna_gqa_prefill: query heads (%d) must be a positive multiple of kv heads (%d)", q_heads, kv_heads);
  ANNA_REQUIRE(q_len > 0 && key_len >= 0, "anna_gqa_prefill: bad lengths (q_len %d, key_len %lld)", q_len,
               (long long)key_len);
  ANNA_REQUIRE(batch <= 65535 && q_heads <= 65535, "anna_gqa_prefill: batch and heads are limited to 65535");
  if (dtype != ANNA_DTYPE_F16 && dtype != ANNA_DTYPE_BF16)
    return set_error(ANNA_ERR_UNSUPPORTED, "anna_gqa_prefill: 16-bit dtypes only (got dtype code %d)", dtype);
  if (head_dim != 64 && head_dim != 128 && head_dim != 256)
    return set_error(ANNA_ERR_UNSUPPORTED, "anna_gqa_prefill: head_dim %d (64, 128 and 256 are built)", head_dim);
  // 16-byte copies: every row start has to be 16-byte aligned
  const int64_t strides[] = {q_stride_b, q_stride_h, q_stride_t, kv_stride_b, kv_stride_h, kv_stride_t};
  for (int64_t s : strides) ANNA_REQUIRE(s % 8 == 0, "anna_gqa_prefill: q / k / v strides must be multiples of 8 elements");
  ANNA_REQUIRE(out_stride_b % 2 == 0 && out_stride_h % 2 == 0 && out_stride_t % 2 == 0,
               "anna_gqa_prefill: output strides must be even");
  ANNA_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)key % 16 == 0 && (uintptr_t)value % 16 == 0 && (uintptr_t)out % 4 == 0,
               "anna_gqa_prefill: q / k / v must be 16-byte aligned");
  PrefillParams p{};
  p.q = q; p.k = key; p.v = value; p.out = out; p.key_lengths = key_lengths;
  p.q_stride_b = q_stride_b; p.q_stride_h = q_stride_h; p.q_stride_t = q_stride_t;
  p.kv_stride_b = kv_stride_b; p.kv_stride_h = kv_stride_h; p.kv_stride_t = kv_stride_t;
  p.out_stride_b = out_stride_b; p.out_stride_h = out_stride_h; p.out_stride_t = out_stride_t;
  p.q_len = q_len; p.groups = q_heads / kv_heads; p.causal = causal != 0;
  p.key_len = key_len;
  p.scale_log2 = scaling * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  if (prefill_umma_applicable(p, head_dim, dtype)) {
    const int rc = launch_prefill_umma(p, batch, q_heads, head_dim, dtype, s);
    if (rc != kPrefillNotServed) return rc;
  }
#define ANNA_PREFILL_CASE(TYPE, DIM) \
  if (head_dim == DIM) return launch_prefill<TYPE, DIM>(p, batch, q_heads, s);
  if (dtype == ANNA_DTYPE_BF16) {
    ANNA_PREFILL_CASE(__nv_bfloat16, 64) ANNA_PREFILL_CASE(__nv_bfloat16, 128) ANNA_PREFILL_CASE(__nv_bfloat16, 256)
  } else {
    ANNA_PREFILL_CASE(__half, 64) ANNA_PREFILL_CASE(__half, 128) ANNA_PREFILL_CASE(__half, 256)
  }
#undef ANNA_PREFILL_CASE
  return set_error(ANNA_ERR_UNSUPPORTED, "anna_gqa_prefill: unsupported head_dim %d", head_dim);
}
