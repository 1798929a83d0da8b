// CUDA-core building blocks for single-token GQA decode with split-K partials.
//
// One CTA (4 warps) owns one (batch row, kv head, context chunk) and every query head of that kv head's group, so
// each K/V byte is read from HBM once per group.  A token row is spread over LPT lanes in 16-byte pieces; a warp
// covers TPW = 32 / LPT tokens per load instruction and keeps U loads in flight.  Scores are reduced with xor
// shuffles inside the LPT-lane team, the softmax is kept online per team in fp32, and the teams of a CTA are merged
// through shared memory before one partial (max, denom, D values) per query head is written out.
#pragma once

#include "common.cuh"

namespace anna {

constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kUnroll = 4;

template <typename T, int D, int G>
struct DecodeCfg {
  static constexpr int kVec = ElemTraits<T>::kVec;
  static constexpr int kPieces = D / kVec;                      // 16-byte pieces per token row
  static constexpr int kLpt = kPieces > 32 ? 32 : kPieces;      // lanes per token
  static constexpr int kCh = kPieces > 32 ? kPieces / 32 : 1;   // pieces per lane
  static constexpr int kTpw = 32 / kLpt;                        // tokens per warp per load
  static constexpr int kDpl = kVec * kCh;                       // dims per lane
  static constexpr int kTeams = kDecodeWarps * kTpw;            // independent softmax teams per CTA
  static_assert(D % kVec == 0, "head_dim must be a multiple of the 16-byte vector width");
  static_assert(kPieces <= 32 || kPieces % 32 == 0, "unsupported head_dim");
};

// Per-lane running state for G query heads.
template <typename T, int D, int G>
struct TeamState {
  using Cfg = DecodeCfg<T, D, G>;
  float q[G][Cfg::kDpl];    // query slice, pre-multiplied by the softmax scaling
  float acc[G][Cfg::kDpl];  // un-normalised output slice
  float m[G];               // running max
  float l[G];               // running denominator

  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.0f;
#pragma unroll
      for (int i = 0; i < Cfg::kDpl; ++i) acc[g][i] = 0.0f;
    }
  }
};

// dim index of element i of this lane's slice
template <typename Cfg>
__device__ __forceinline__ int lane_dim(int dl, int i) {
  const int piece = i / Cfg::kVec;
  return (piece * Cfg::kLpt + dl) * Cfg::kVec + (i % Cfg::kVec);
}

// Load this lane's query slices (already rotated / scaled queries come from shared memory as float).
template <typename T, int D, int G>
__device__ __forceinline__ void load_query_from_smem(TeamState<T, D, G>& st, const float* __restrict__ q_smem,
                                                     int dl, float scale) {
  using Cfg = DecodeCfg<T, D, G>;
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < Cfg::kDpl; ++i) st.q[g][i] = q_smem[g * D + lane_dim<Cfg>(dl, i)] * scale;
}

// One batch of U tokens per team: tokens are described by element offsets (or -1 for "no token").
// k_base / v_base point at token offset 0 of this (row, kv head).
template <typename T, int D, int G>
__device__ __forceinline__ void team_consume(TeamState<T, D, G>& st, const T* __restrict__ k_base,
                                             const T* __restrict__ v_base, const int64_t (&off)[kUnroll], int dl) {
  using Cfg = DecodeCfg<T, D, G>;
  uint4 kraw[kUnroll][Cfg::kCh];
  uint4 vraw[kUnroll][Cfg::kCh];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
    for (int c = 0; c < Cfg::kCh; ++c) {
      if (off[u] >= 0) {
        kraw[u][c] = ldg_stream16(k_base + off[u] + (c * Cfg::kLpt + dl) * Cfg::kVec);
      } else {
        kraw[u][c] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
    for (int c = 0; c < Cfg::kCh; ++c) {
      if (off[u] >= 0) {
        vraw[u][c] = ldg_stream16(v_base + off[u] + (c * Cfg::kLpt + dl) * Cfg::kVec);
      } else {
        vraw[u][c] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }

  float s[kUnroll][G];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    float kf[Cfg::kDpl];
#pragma unroll
    for (int c = 0; c < Cfg::kCh; ++c) {
      float piece[Cfg::kVec];
      widen16<T>(kraw[u][c], piece);
#pragma unroll
      for (int i = 0; i < Cfg::kVec; ++i) kf[c * Cfg::kVec + i] = piece[i];
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < Cfg::kDpl; ++i) dot = fmaf(st.q[g][i], kf[i], dot);
      s[u][g] = dot;
    }
  }
#pragma unroll
  for (int d = Cfg::kLpt / 2; d >= 1; d >>= 1) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int g = 0; g < G; ++g) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], d);
  }

  float p[kUnroll][G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float m_new = st.m[g];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (off[u] < 0) s[u][g] = -INFINITY;
      m_new = fmaxf(m_new, s[u][g]);
    }
    const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
    const float rescale = __expf(st.m[g] - m_safe);  // exp(-inf) = 0 on the first batch
    float lsum = st.l[g] * rescale;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      p[u][g] = __expf(s[u][g] - m_safe);
      lsum += p[u][g];
    }
    st.l[g] = lsum;
    st.m[g] = m_new;
#pragma unroll
    for (int i = 0; i < Cfg::kDpl; ++i) st.acc[g][i] *= rescale;
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    float vf[Cfg::kDpl];
#pragma unroll
    for (int c = 0; c < Cfg::kCh; ++c) {
      float piece[Cfg::kVec];
      widen16<T>(vraw[u][c], piece);
#pragma unroll
      for (int i = 0; i < Cfg::kVec; ++i) vf[c * Cfg::kVec + i] = piece[i];
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < Cfg::kDpl; ++i) st.acc[g][i] = fmaf(p[u][g], vf[i], st.acc[g][i]);
  }
}

// Merge the teams of a CTA and write one partial per query head.
//   smem needs kTeams * G * (D + 2) floats.
template <typename T, int D, int G>
__device__ __forceinline__ void cta_merge_store(const TeamState<T, D, G>& st, float* __restrict__ smem, int warp,
                                                int sub, int dl, int g_count, float* __restrict__ stats_out,
                                                float* __restrict__ values_out, int64_t head_stride_stats,
                                                int64_t head_stride_values) {
  using Cfg = DecodeCfg<T, D, G>;
  const int team = warp * Cfg::kTpw + sub;
  float* sm_m = smem;                         // [teams][G]
  float* sm_l = smem + Cfg::kTeams * G;       // [teams][G]
  float* sm_acc = smem + 2 * Cfg::kTeams * G; // [teams][G][D]
  if (dl == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      sm_m[team * G + g] = st.m[g];
      sm_l[team * G + g] = st.l[g];
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < Cfg::kDpl; ++i) sm_acc[(team * G + g) * D + lane_dim<Cfg>(dl, i)] = st.acc[g][i];
  __syncthreads();
  for (int item = threadIdx.x; item < g_count * D; item += kDecodeThreads) {
    const int g = item / D;
    const int d = item % D;
    float m_all = -INFINITY;
#pragma unroll
    for (int t = 0; t < Cfg::kTeams; ++t) m_all = fmaxf(m_all, sm_m[t * G + g]);
    const float m_safe = (m_all == -INFINITY) ? 0.0f : m_all;
    float l_all = 0.0f, a_all = 0.0f;
#pragma unroll
    for (int t = 0; t < Cfg::kTeams; ++t) {
      const float w = __expf(sm_m[t * G + g] - m_safe);
      l_all += sm_l[t * G + g] * w;
      a_all += sm_acc[(t * G + g) * D + d] * w;
    }
    values_out[g * head_stride_values + d] = a_all;
    if (d == 0) {
      stats_out[g * head_stride_stats + 0] = m_all;
      stats_out[g * head_stride_stats + 1] = l_all;
    }
  }
}

// Host-side dispatch helpers -------------------------------------------------------------------------------------

inline int padded_group(int g) { return g <= 1 ? 1 : (g <= 2 ? 2 : (g <= 4 ? 4 : 8)); }

#define ANNA_DISPATCH_DIM(dim, D, ...)                                                       \
  [&]() -> int {                                                                             \
    switch (dim) {                                                                           \
      case 64: { constexpr int D = 64; return __VA_ARGS__(); }                               \
      case 128: { constexpr int D = 128; return __VA_ARGS__(); }                             \
      case 256: { constexpr int D = 256; return __VA_ARGS__(); }                             \
      default: return ::anna::set_error(ANNA_ERR_UNSUPPORTED, "unsupported head_dim %d (64, 128, 256)", (int)(dim)); \
    }                                                                                        \
  }()

#define ANNA_DISPATCH_GROUP(gpad, G, ...)                                                    \
  [&]() -> int {                                                                             \
    switch (gpad) {                                                                          \
      case 1: { constexpr int G = 1; return __VA_ARGS__(); }                                 \
      case 2: { constexpr int G = 2; return __VA_ARGS__(); }                                 \
      case 4: { constexpr int G = 4; return __VA_ARGS__(); }                                 \
      default: { constexpr int G = 8; return __VA_ARGS__(); }                                \
    }                                                                                        \
  }()

}  // namespace anna
