// Second pass of split-K decode: merge the per-chunk partials of each (row, query head), apply the optional
// sigmoid(gate) epilogue and store in the query dtype.  Also holds the library-wide error plumbing.
#include <cstring>

#include "decode_core.cuh"

namespace anna {

static thread_local char g_last_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
  va_end(args);
  return code;
}

struct CombineParams {
  const float* stats;
  const float* values;
  const int32_t* lengths32;
  const int64_t* lengths64;
  int64_t fixed_len, max_len;
  int window;  // > 0: chunks = ceil(min(L, window) / c) + ceil(max(L - window, 0) / c)
  const void* gate;
  int64_t gate_stride_b, gate_stride_h;
  void* out;
  int64_t out_stride_b, out_stride_h;
  int q_heads, head_dim, chunk_tokens, num_chunks, chunk_capacity;
};

template <typename T>
__global__ void __launch_bounds__(128) split_combine_kernel(const CombineParams p) {
  const int h = blockIdx.x;
  const int b = blockIdx.y;
  int64_t len = p.lengths32 ? (int64_t)p.lengths32[b] : (p.lengths64 ? p.lengths64[b] : p.fixed_len);
  len = max((int64_t)0, min(len, p.max_len));
  int chunks;
  if (p.window > 0) {
    const int64_t win = min(len, (int64_t)p.window);
    chunks = (int)((win + p.chunk_tokens - 1) / p.chunk_tokens + (len - win + p.chunk_tokens - 1) / p.chunk_tokens);
  } else {
    chunks = (int)((len + p.chunk_tokens - 1) / p.chunk_tokens);
  }
  const int64_t part = ((int64_t)b * p.q_heads + h) * p.chunk_capacity;
  const float* stats = p.stats + part * 2;
  const float* values = p.values + part * p.head_dim;

  __shared__ float sm_max[4];
  __shared__ float sm_den[4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  float m = -INFINITY;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) m = fmaxf(m, stats[2 * c]);
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  if (lane == 0) sm_max[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(sm_max[0], sm_max[1]), fmaxf(sm_max[2], sm_max[3]));
  const float m_safe = (m == -INFINITY) ? 0.0f : m;

  float den = 0.0f;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) den += stats[2 * c + 1] * __expf(stats[2 * c] - m_safe);
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) den += __shfl_xor_sync(0xffffffffu, den, d);
  if (lane == 0) sm_den[warp] = den;
  __syncthreads();
  den = (sm_den[0] + sm_den[1]) + (sm_den[2] + sm_den[3]);
  const float inv = den > 0.0f ? 1.0f / den : 0.0f;

  T* out = reinterpret_cast<T*>(p.out) + (int64_t)b * p.out_stride_b + (int64_t)h * p.out_stride_h;
  const T* gate = p.gate ? reinterpret_cast<const T*>(p.gate) + (int64_t)b * p.gate_stride_b +
                               (int64_t)h * p.gate_stride_h
                         : nullptr;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) {
    float acc = 0.0f;
    for (int c = 0; c < chunks; ++c) acc = fmaf(values[(int64_t)c * p.head_dim + d], __expf(stats[2 * c] - m_safe), acc);
    float v = acc * inv;
    if (gate) v *= sigmoidf_fast(ElemTraits<T>::to_float(gate[d]));
    out[d] = ElemTraits<T>::from_float(v);
  }
}

int resolve_split(int batch, int kv_heads, int64_t max_len, int chunk_tokens_in, int chunk_capacity,
                  const float* partial_stats, const float* partial_values, int* chunk_tokens, int* num_chunks) {
  if (partial_stats == nullptr || partial_values == nullptr)
    return set_error(ANNA_ERR_WORKSPACE, "decode needs partial_stats and partial_values scratch buffers");
  if (chunk_tokens_in > 0) {
    const int64_t chunks = max_len > 0 ? (max_len + chunk_tokens_in - 1) / chunk_tokens_in : 1;
    if (chunks > 65535 * 16) return set_error(ANNA_ERR_INVALID, "too many split-K chunks (%lld)", (long long)chunks);
    *chunk_tokens = chunk_tokens_in;
    *num_chunks = (int)chunks;
  } else {
    const int rc = anna_decode_plan(batch, kv_heads, max_len, chunk_tokens, num_chunks);
    if (rc != ANNA_OK) return rc;
  }
  if (*num_chunks > chunk_capacity)
    return set_error(ANNA_ERR_WORKSPACE, "split-K scratch holds %d chunks per head, %d needed", chunk_capacity,
                     *num_chunks);
  return ANNA_OK;
}

int launch_split_combine(const SplitWorkspace& ws, const int32_t* lengths32, const int64_t* lengths64,
                         int64_t fixed_len, int64_t max_len, int window, const void* gate, int64_t gate_stride_b,
                         int64_t gate_stride_h, void* out, int64_t out_stride_b, int64_t out_stride_h, int batch,
                         int q_heads, int head_dim, int chunk_tokens, int num_chunks, int dtype,
                         cudaStream_t stream) {
  CombineParams p{};
  p.stats = ws.stats; p.values = ws.values;
  p.lengths32 = lengths32; p.lengths64 = lengths64; p.fixed_len = fixed_len; p.max_len = max_len; p.window = window;
  p.gate = gate; p.gate_stride_b = gate_stride_b; p.gate_stride_h = gate_stride_h;
  p.out = out; p.out_stride_b = out_stride_b; p.out_stride_h = out_stride_h;
  p.q_heads = q_heads; p.head_dim = head_dim; p.chunk_tokens = chunk_tokens; p.num_chunks = num_chunks;
  p.chunk_capacity = ws.chunk_capacity;
  dim3 grid((unsigned)q_heads, (unsigned)batch);
  return ANNA_DISPATCH_DTYPE(dtype, T, [&]() -> int {
    split_combine_kernel<T><<<grid, 128, 0, stream>>>(p);
    return check_launch("split_combine_kernel");
  });
}

}  // namespace anna

extern "C" const char* anna_kv_last_error(void) { return anna::g_last_error; }
extern "C" int anna_kv_abi_version(void) { return 1; }
