// Fused TurboQuant append: residual-window ring update + quantize-on-overflow + bit-pack + page scatter.
//
// One warp owns one (row, kv head, token) work item.  Items of a row with old length L, T new tokens, window R:
//   quantize items  p in [max(0, L-R), max(0, L+T-R)) : source is the ring (p < L) or the incoming chunk (p >= L)
//   window items    p in [max(L, L+T-R), L+T)         : incoming token copied into ring slot p % R
// A ring slot that is both read (old token being quantized) and written (new token with the same residue) in one
// call is handled by the reading warp: it loads the old vectors into registers, then stores the new ones.
#include "tq_common.cuh"

namespace anna {

struct TqAppendParams {
  const void* k_new;
  const void* v_new;
  int64_t stride_b, stride_h, stride_t;
  uint8_t* pages;
  const int32_t* block_table;
  int64_t table_stride;
  const uint32_t* shared_blocks;  // optional bit mask [batch, mask_stride words]: block already holds these tokens
  int64_t mask_stride;
  void* window;
  const int64_t* window_slots;
  const int64_t* old_lengths;
  int64_t* new_lengths;
  const float* signs1;
  const float* signs2;
  const float* centroids;
  const float* boundaries;
  int batch, kv_heads, new_tokens, block_size, residual_len, value_group;
  int block_shift, residual_shift;  // log2 when the value is a power of two, else -1
  int u_chunks;                     // CTAs along the item axis of one (row, kv head)
  int64_t num_pages, max_blocks;
  anna_tq_layout layout;
  int32_t* status;
};

constexpr int kAppendWarps = 8;

// Number of boundaries below `s` (= index of the nearest centroid) by bisection over the sorted boundaries: three
// compares for 7 boundaries instead of seven.  Same result as counting `s > bnd[k]` over all k, NaN included (0).
template <int NB>
__device__ __forceinline__ uint32_t codebook_index(float s, const float (&bnd)[NB]) {
  if constexpr (NB == 1) {
    return s > bnd[0] ? 1u : 0u;
  } else if constexpr (NB == 3) {
    const bool p0 = s > bnd[1];
    const bool p1 = s > (p0 ? bnd[2] : bnd[0]);
    return (p0 ? 2u : 0u) + (p1 ? 1u : 0u);
  } else {
    static_assert(NB == 7, "codebooks have 2, 4 or 8 entries");
    const bool p0 = s > bnd[3];
    const bool p1 = s > (p0 ? bnd[5] : bnd[1]);
    const float upper = p1 ? bnd[6] : bnd[4], lower = p1 ? bnd[2] : bnd[0];
    const bool p2 = s > (p0 ? upper : lower);
    return (p0 ? 4u : 0u) + (p1 ? 2u : 0u) + (p2 ? 1u : 0u);
  }
}

// a / s, correctly rounded, from y = RN(1 / s): one multiply and two fused multiply-adds.  Exact (Markstein) while
// nothing over- or underflows and the significand of s is not all ones; callers fall back to the division otherwise.
__device__ __forceinline__ float div_by_shared(float a, float s, float y) {
  const float q0 = __fmul_rn(a, y);
  return __fmaf_rn(__fmaf_rn(-q0, s, a), y, q0);
}

// A CTA belongs to one (row, kv head); its warps stride over that head's 2 * new_tokens items, so everything that does
// not depend on the item -- sign vectors, boundaries, centroids, lengths, ring and pool bases -- is set up once per
// warp.  Positions are 32-bit (the host rejects longer contexts) and divisions by the window length and the page size
// are shifts when those are powers of two.
template <typename T, int D, int BITS>
__global__ void __launch_bounds__(kAppendWarps * 32) tq_append_kernel(const TqAppendParams p) {
  constexpr int E = D / 32;
  constexpr int M = BITS - 1;          // index bits
  constexpr int NB = (1 << M) - 1;     // boundaries
  constexpr int VS = BITS == 2 ? 2 : 4;  // value storage bits
  __shared__ float sm_cent[1 << M];
  if (threadIdx.x < (1 << M)) sm_cent[threadIdx.x] = p.centroids[threadIdx.x];
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int e0 = lane * E;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  // bit j: coordinate e0 + j is negated by the rotation (low byte) / by the QJL projection (next byte)
  uint32_t flips = 0;
#pragma unroll
  for (int j = 0; j < E; ++j) {
    flips |= (p.signs1[e0 + j] < 0.0f ? 1u : 0u) << j;
    flips |= (p.signs2[e0 + j] < 0.0f ? 1u : 0u) << (8 + j);
  }
  float bnd[NB];
#pragma unroll
  for (int k = 0; k < NB; ++k) bnd[k] = p.boundaries[k];
  constexpr float rsqrt_dim = rsqrt_dim_const<D>();
  const float levels = (float)((1 << BITS) - 1);
  const float inv_levels = __frcp_rn(levels);
  const int lanes_per_group = p.value_group / E;  // power of two, >= 1
  const int R = p.residual_len;
  const int Tn = p.new_tokens;
  const int S = p.block_size;
  auto div_r = [&](int v) { return p.residual_shift >= 0 ? v >> p.residual_shift : v / R; };
  auto div_s = [&](int v) { return p.block_shift >= 0 ? v >> p.block_shift : v / S; };

  const int L = (int)p.old_lengths[b];
  const int Lp = L + Tn;
  if (p.new_lengths != nullptr && (blockIdx.x | blockIdx.y | threadIdx.x) == 0) p.new_lengths[b] = Lp;
  const int Lq = L > R ? L - R : 0;
  const int Lqp = Lp > R ? Lp - R : 0;
  const int nq = Lqp - Lq;
  const int wstart = L > Lqp ? L : Lqp;
  const int nw = Lp - wstart;
  const int64_t slot = p.window_slots[b];
  T* ring_k = reinterpret_cast<T*>(p.window) + ((slot * 2 + 0) * p.kv_heads + h) * (int64_t)R * D + e0;
  T* ring_v = reinterpret_cast<T*>(p.window) + ((slot * 2 + 1) * p.kv_heads + h) * (int64_t)R * D + e0;
  // incoming token at position pos sits at in_k + (pos - L) * stride_t
  const T* in_k = reinterpret_cast<const T*>(p.k_new) + (int64_t)b * p.stride_b + (int64_t)h * p.stride_h + e0;
  const T* in_v = reinterpret_cast<const T*>(p.v_new) + (int64_t)b * p.stride_b + (int64_t)h * p.stride_h + e0;
  const int32_t* table_row = p.block_table + (int64_t)b * p.table_stride;

  const int warp = threadIdx.x >> 5;
  const int u_stride = p.u_chunks * kAppendWarps;

  // ---- window items: plain copies, unless the slot's old occupant is quantized (and rewritten) by a quantize item ----
  for (int u = (int)blockIdx.x * kAppendWarps + warp; u < nw; u += u_stride) {
    const int pw = wstart + u;
    const int k = div_r(pw - L + R);  // smallest k >= 1 with pw - k*R < L
    const int p_old = pw - k * R;
    if (p_old >= Lq) continue;
    const int rs = pw - div_r(pw) * R;
    lane_copy<T, E>(in_k + (int64_t)(pw - L) * p.stride_t, ring_k + rs * D);
    lane_copy<T, E>(in_v + (int64_t)(pw - L) * p.stride_t, ring_v + rs * D);
  }

  // ---- quantize items.  The trip count depends on the CTA alone, so every warp stays converged through the warp
  // exchanges of the body; a warp past the end repeats the last item and stores nothing. ------------------------------
  for (int base = (int)blockIdx.x * kAppendWarps; base < nq; base += u_stride) {
    const bool active = base + warp < nq;
    const int pos = Lq + (active ? base + warp : nq - 1);
    float x[E], v[E];
    if (pos < L) {
      const int rs = pos - div_r(pos) * R;
      lane_load<T, E>(ring_k + rs * D, x);
      lane_load<T, E>(ring_v + rs * D, v);
      const int k = div_r(wstart - pos + R - 1);
      const int pw = pos + k * R;  // new occupant of this ring slot, if it arrives in this call
      if (active && pw < Lp) {
        lane_copy<T, E>(in_k + (int64_t)(pw - L) * p.stride_t, ring_k + rs * D);
        lane_copy<T, E>(in_v + (int64_t)(pw - L) * p.stride_t, ring_v + rs * D);
      }
    } else {
      lane_load<T, E>(in_k + (int64_t)(pos - L) * p.stride_t, x);
      lane_load<T, E>(in_v + (int64_t)(pos - L) * p.stride_t, v);
    }

    const int blk = div_s(pos);
    const int tok = pos - blk * S;
    int32_t pid = -1;
    if (blk < p.max_blocks) pid = table_row[blk];
    bool store = active;
    if (pid < 0 || pid >= p.num_pages) {
      if (active && lane == 0 && p.status) atomicOr(p.status, (int)ANNA_DEV_BAD_PAGE);
      store = false;
      pid = 0;
    }
    // a block mapped from another sequence with the same prompt prefix already holds exactly these codes
    if (p.shared_blocks != nullptr && ((p.shared_blocks[(int64_t)b * p.mask_stride + (blk >> 5)] >> (blk & 31)) & 1u))
      store = false;
    uint8_t* chunk = p.pages + ((int64_t)pid * p.kv_heads + h) * p.layout.chunk_bytes;

    // ---- keys: normalise, rotate, index, residual sign ----------------------------------------------------------
    float t[E], w[E];
#pragma unroll
    for (int j = 0; j < E; ++j) t[j] = __fmul_rn(x[j], x[j]);
    const float norm = __fsqrt_rn(warp_tree_sum<E>(t));
    const float inv = __frcp_rn(fmaxf(norm, 1e-20f));
#pragma unroll
    for (int j = 0; j < E; ++j) w[j] = __uint_as_float(__float_as_uint(x[j]) ^ ((flips >> j) << 31));
    warp_fwht<E>(w, lane);

    uint32_t code[E];
    float e[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float scaled = __fmul_rn(w[j], inv);
      const uint32_t c = codebook_index<NB>(scaled, bnd);
      code[j] = c;
      e[j] = __fsub_rn(scaled, sm_cent[c]);
    }
#pragma unroll
    for (int j = 0; j < E; ++j) t[j] = __fmul_rn(e[j], e[j]);
    const float rnorm = __fmul_rn(__fsqrt_rn(warp_tree_sum<E>(t)), rsqrt_dim);
#pragma unroll
    for (int j = 0; j < E; ++j) e[j] = __uint_as_float(__float_as_uint(e[j]) ^ ((flips >> (8 + j)) << 31));
    warp_fwht<E>(e, lane);

    uint8_t* krow = chunk + p.layout.off_kcodes + tok * p.layout.key_bytes;
    if constexpr (BITS == 4) {
      uint64_t field = 0;
#pragma unroll
      for (int j = 0; j < E; ++j) field |= (uint64_t)(code[j] | (e[j] >= 0.0f ? 8u : 0u)) << (4 * j);
      warp_pack_store<4 * E>(field, krow, lane, store);
    } else if constexpr (BITS == 2) {
      uint64_t field = 0;
#pragma unroll
      for (int j = 0; j < E; ++j) field |= (uint64_t)(code[j] | (e[j] >= 0.0f ? 2u : 0u)) << (2 * j);
      warp_pack_store<2 * E>(field, krow, lane, store);
    } else {
      uint64_t idx_field = 0, sign_field = 0;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        idx_field |= (uint64_t)code[j] << (2 * j);
        sign_field |= (uint64_t)(e[j] >= 0.0f ? 1u : 0u) << j;
      }
      warp_pack_store<2 * E>(idx_field, krow, lane, store);
      warp_pack_store<E>(sign_field, krow + D / 4, lane, store);
    }
    if (store && lane == 0) {
      reinterpret_cast<float*>(chunk + p.layout.off_knorm)[tok] = norm;
      reinterpret_cast<float*>(chunk + p.layout.off_krnorm)[tok] = rnorm;
    }

    // ---- values: per-group min/max -> scale / zero in the cache dtype -> round-half-even codes -------------------
    float lo = v[0], hi = v[0];
#pragma unroll
    for (int j = 1; j < E; ++j) {
      lo = fminf(lo, v[j]);
      hi = fmaxf(hi, v[j]);
    }
#pragma unroll
    for (int dl = 1; dl < 32; dl <<= 1) {
      if (dl < lanes_per_group) {  // uniform over the grid
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, dl));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, dl));
      }
    }
    // The divisions below share their divisor inside a group (the scale) or over the whole launch (the level count),
    // so each is a reciprocal taken once and a three-instruction correction per quotient; operands outside the safe
    // range (an infinite or NaN range, a scale that rounds to zero in the cache dtype, fp32 caches whose scale can
    // have any significand) take the plain correctly rounded division.
    const float range = __fsub_rn(hi, lo);
    const bool tame = sizeof(T) == 2 && range < 1e30f;
    const float raw = tame ? div_by_shared(range, levels, inv_levels) : __fdiv_rn(range, levels);
    const float scale = round_to_elem<T>(raw < 1e-8f ? 1e-8f : raw);
    const float zero = round_to_elem<T>(lo);
    uint64_t vfield = 0;
    if (tame && scale >= 1e-9f) {
      const float inv_scale = __frcp_rn(scale);
#pragma unroll
      for (int j0 = 0; j0 < E; j0 += 4) {
        // four codes (at most 16 bits) are packed as an exact fp32 sum before the one conversion to integer
        float packed = 0.0f;
#pragma unroll
        for (int j = j0; j < j0 + 4 && j < E; ++j) {
          float q = rintf(div_by_shared(__fsub_rn(v[j], zero), scale, inv_scale));
          q = fminf(fmaxf(q, 0.0f), levels);  // a NaN becomes 0, as in `if (!(q >= 0)) q = 0`
          packed = __fmaf_rn(q, (float)(1u << (VS * (j - j0))), packed);
        }
        vfield |= (uint64_t)(uint32_t)packed << (VS * j0);
      }
    } else {
#pragma unroll
      for (int j = 0; j < E; ++j) {
        float q = rintf(__fdiv_rn(__fsub_rn(v[j], zero), scale));
        if (!(q >= 0.0f)) q = 0.0f;
        if (q > levels) q = levels;
        vfield |= (uint64_t)(uint32_t)q << (VS * j);
      }
    }
    warp_pack_store<VS * E>(vfield, chunk + p.layout.off_vdata + tok * p.layout.value_bytes, lane, store);
    if (store && lane % lanes_per_group == 0) {
      const int g = lane / lanes_per_group;
      reinterpret_cast<T*>(chunk + p.layout.off_vscale)[tok * p.layout.groups + g] = ElemTraits<T>::from_float(scale);
      reinterpret_cast<T*>(chunk + p.layout.off_vzero)[tok * p.layout.groups + g] = ElemTraits<T>::from_float(zero);
    }
  }
}

}  // namespace anna

using namespace anna;

extern "C" int anna_tq_page_layout(int head_dim, int bits, int block_size, int dtype, int value_group,
                                   anna_tq_layout* out) {
  ANNA_REQUIRE(out != nullptr, "anna_tq_page_layout: null output");
  ANNA_REQUIRE(dtype >= 0 && dtype <= 2, "anna_tq_page_layout: bad dtype code %d", dtype);
  if (!tq_make_layout(head_dim, bits, block_size, dtype_bytes_of(dtype), value_group, out))
    return set_error(ANNA_ERR_INVALID, "anna_tq_page_layout: unsupported geometry D=%d bits=%d S=%d group=%d", head_dim,
                     bits, block_size, value_group);
  return ANNA_OK;
}

extern "C" int anna_tq_append(const void* k_new, const void* v_new, int64_t kn_stride_b, int64_t kn_stride_h,
                              int64_t kn_stride_t, uint8_t* packed_pages, const int32_t* block_table,
                              int64_t table_stride, const uint32_t* shared_blocks, int64_t mask_stride, void* window, const int64_t* window_slots,
                              const int64_t* old_lengths, int64_t* new_lengths, const float* signs1,
                              const float* signs2, const float* centroids, const float* boundaries, int batch, int kv_heads,
                              int new_tokens, int head_dim, int block_size, int residual_len, int bits,
                              int value_group, int64_t num_pages, int64_t max_blocks, int dtype, int32_t* status,
                              anna_stream_t stream) {
  ANNA_REQUIRE(k_new && v_new && window && window_slots && old_lengths && signs1 && signs2 && centroids && boundaries,
               "anna_tq_append: null pointer argument");
  ANNA_REQUIRE(new_lengths != old_lengths, "anna_tq_append: new_lengths must not alias old_lengths");
  ANNA_REQUIRE(batch > 0 && kv_heads > 0 && new_tokens > 0 && residual_len >= 1 && block_size >= 1,
               "anna_tq_append: sizes must be positive");
  ANNA_REQUIRE(packed_pages != nullptr || num_pages == 0, "anna_tq_append: null page pool with num_pages > 0");
  ANNA_REQUIRE(block_table != nullptr || max_blocks == 0, "anna_tq_append: null block table with max_blocks > 0");
  const int lane_elems = head_dim / 32;
  ANNA_REQUIRE(lane_elems >= 1 && value_group >= lane_elems && value_group % lane_elems == 0 &&
                   ((value_group / lane_elems) & (value_group / lane_elems - 1)) == 0 && value_group <= head_dim,
               "anna_tq_append: value group %d does not fit head_dim %d", value_group, head_dim);
  const int vec = dtype == ANNA_DTYPE_F32 ? 4 : 8;
  ANNA_REQUIRE(kn_stride_b % vec == 0 && kn_stride_h % vec == 0 && kn_stride_t % vec == 0,
               "anna_tq_append: source strides must keep rows 16-byte aligned");
  TqAppendParams p{};
  p.k_new = k_new; p.v_new = v_new;
  p.stride_b = kn_stride_b; p.stride_h = kn_stride_h; p.stride_t = kn_stride_t;
  p.pages = packed_pages; p.block_table = block_table; p.table_stride = table_stride;
  p.shared_blocks = shared_blocks; p.mask_stride = mask_stride;
  ANNA_REQUIRE(shared_blocks == nullptr || mask_stride * 32 >= max_blocks,
               "anna_tq_append: shared-block mask of %lld words per row does not cover %lld blocks", (long long)mask_stride,
               (long long)max_blocks);
  p.window = window; p.window_slots = window_slots; p.old_lengths = old_lengths; p.new_lengths = new_lengths;
  p.signs1 = signs1; p.signs2 = signs2; p.centroids = centroids; p.boundaries = boundaries;
  p.batch = batch; p.kv_heads = kv_heads; p.new_tokens = new_tokens; p.block_size = block_size;
  p.residual_len = residual_len; p.value_group = value_group;
  p.num_pages = num_pages; p.max_blocks = max_blocks; p.status = status;
  if (!tq_make_layout(head_dim, bits, block_size, dtype_bytes_of(dtype), value_group, &p.layout))
    return set_error(ANNA_ERR_INVALID, "anna_tq_append: unsupported geometry D=%d bits=%d S=%d group=%d", head_dim, bits,
                     block_size, value_group);
  ANNA_REQUIRE((int64_t)new_tokens < ((int64_t)1 << 29) && max_blocks * (int64_t)block_size < ((int64_t)1 << 30),
               "anna_tq_append: context too long for 32-bit positions");
  p.block_shift = p.residual_shift = -1;
  for (int sh = 0; sh < 30; ++sh) {
    if ((1 << sh) == block_size) p.block_shift = sh;
    if ((1 << sh) == residual_len) p.residual_shift = sh;
  }
  return ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    return ANNA_DISPATCH_TQ_DIM(head_dim, D, [&]() -> int {
      return ANNA_DISPATCH_TQ_BITS(bits, BITS, [&]() -> int {
        auto kernel = tq_append_kernel<T, D, BITS>;
        static int resident[64] = {};  // per device: CTAs of this kernel that fit the whole GPU at once
        int device = 0;
        ANNA_CUDA_CHECK(cudaGetDevice(&device));
        int ctas = (device >= 0 && device < 64) ? resident[device] : 0;
        if (ctas == 0) {
          int sms = 0, per_sm = 0;
          ANNA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
          ANNA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kAppendWarps * 32, 0));
          ctas = sms * (per_sm > 0 ? per_sm : 1);
          if (device >= 0 && device < 64) resident[device] = ctas;
        }
        // about two resident waves of CTAs, each (row, kv head) cut into u_chunks pieces along its items
        const int64_t heads_total = (int64_t)kv_heads * batch;
        const int64_t max_chunks = (2 * (int64_t)new_tokens + kAppendWarps - 1) / kAppendWarps;
        int64_t chunks = (2 * (int64_t)ctas + heads_total - 1) / heads_total;
        if (chunks > max_chunks) chunks = max_chunks;
        if (chunks < 1) chunks = 1;
        TqAppendParams q = p;
        q.u_chunks = (int)chunks;
        dim3 grid((unsigned)chunks, (unsigned)kv_heads, (unsigned)batch);
        kernel<<<grid, kAppendWarps * 32, 0, (cudaStream_t)stream>>>(q);
        return check_launch("tq_append_kernel");
      });
    });
  });
}
