// Tensor-core split pass of single-token GQA decode over un-quantized 16-bit K/V (paged or dense strided).
//
// One CTA (4 warps) owns one (row, kv head, context chunk); each warp walks 16-token tiles of the chunk on its own:
//   global --cp.async 16 B, xor-swizzled--> shared (3 stages per warp) --ldmatrix--> mma.sync m16n8k16
//   S[16 tok x 8 heads]   = K_tile[16 x D] . Q^T[D x 8]            (D/16 MMAs, Q^T fragments live in registers)
//   online softmax in fp32 on the C fragments, lazily rescaled; P packed to 16 bit and transposed with movmatrix
//   O^T[D x 8 heads]     += V_tile^T[D x 16] . P^T[16 x 8]          (D/16 MMAs, V^T through ldmatrix.trans)
// The 8 columns are the query heads of the kv head's group (zero padded), so each K/V byte leaves HBM once per group
// and is touched by no CUDA-core instruction.  Every warp keeps its own (max, sum, O) and the four are merged through
// shared memory into one split-K partial per query head.
#include "dense_mma_body.cuh"

#include <cstdlib>

namespace anna {

template <typename T, int D>
__global__ void __launch_bounds__(kMmaThreads, MmaCfg<D>::kMinBlocks)
dense_decode_split_mma_kernel(const DenseDecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int chunk = blockIdx.x;
  const int group_tiles = (p.groups + 7) / 8;
  const int kvh = blockIdx.y / group_tiles;
  const int g0 = (blockIdx.y % group_tiles) * 8;
  const int g_count = min(8, p.groups - g0);
  const int b = blockIdx.z;

  int64_t len64 = p.visible_lengths ? p.visible_lengths[b] : p.max_len;
  len64 = max((int64_t)0, min(len64, p.max_len));
  const int64_t t0_64 = (int64_t)chunk * p.chunk_tokens;
  if (t0_64 >= len64) {
    if (p.fused.counters != nullptr && chunk == 0)  // empty row: nobody else will write its output
      fused_write_zero_row<T, D, kMmaThreads>(p.fused, b, kvh * p.groups + g0, g_count);
    return;
  }
  // all token positions fit 31 bits (the host rejects longer contexts)
  const int t0 = (int)t0_64;
  const int t1 = (int)min(len64, t0_64 + p.chunk_tokens);
  const int active_chunks = (int)((len64 + p.chunk_tokens - 1) / p.chunk_tokens);
  dense_split_mma_body<T, D>(p, smem_raw, b, kvh, g0, g_count, t0, t1, chunk, active_chunks,
                             (int64_t)b * gridDim.y + blockIdx.y);
}

// ---------------------------------------------------------------------------------------------------------------------
// Balanced persistent variant.  The 16-token tiles of all (row, kv head, group-of-8) streams form one line, in
// (row, stream-in-row, tile) order; the grid is one resident wave and CTA c owns tiles [c * tpc, (c + 1) * tpc).  A CTA
// walks its range stream by stream and emits one split-K partial per stream it touches, so every CTA moves the same
// number of bytes whatever the mix of context lengths, and a long context costs one pipeline start per CTA, not one
// per fixed-size chunk.  The partition is recomputed by every CTA from the device-side lengths (a 128-thread scan),
// so no host round trip is needed; slot numbers and arrival counts for the fused merge follow from the same arithmetic.
constexpr int kBalancedMaxRows = 1024;
constexpr int kBalancedMinTiles = 4;  // one tile per warp

template <typename T, int D>
__global__ void __launch_bounds__(kMmaThreads, MmaCfg<D>::kMinBlocks)
dense_decode_balanced_mma_kernel(const DenseDecodeParams p, const int batch) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ int s_prefix[kBalancedMaxRows + 1];  // tiles (over all streams) of the rows before row b
  __shared__ int s_warp_sum[kMmaWarps];
  __shared__ int s_warp_max[kMmaWarps];

  const int group_tiles = (p.groups + 7) / 8;
  const int streams_per_row = p.kv_heads * group_tiles;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  auto row_len = [&](int b) -> int {
    int64_t len = p.visible_lengths ? p.visible_lengths[b] : p.max_len;
    return (int)max((int64_t)0, min(len, p.max_len));
  };

  // ---- exclusive scan of tiles per row ------------------------------------------------------------------------------
  constexpr int kRowsPerThread = kBalancedMaxRows / kMmaThreads;
  const int rpt = (batch + kMmaThreads - 1) / kMmaThreads;
  int local[kRowsPerThread];
  int sum = 0, mx = 0;
#pragma unroll
  for (int i = 0; i < kRowsPerThread; ++i) {
    const int b = threadIdx.x * rpt + i;
    local[i] = (i < rpt && b < batch) ? (row_len(b) + kTileTokens - 1) / kTileTokens : 0;
    sum += local[i];
    mx = max(mx, local[i]);
  }
  int incl = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  }
  if (lane == 31) s_warp_sum[warp] = incl;
  if (lane == 0) s_warp_max[warp] = mx;
  __syncthreads();
  int excl = incl - sum;
  int total = 0, max_tiles = 0;
#pragma unroll
  for (int w = 0; w < kMmaWarps; ++w) {
    if (w < warp) excl += s_warp_sum[w];
    total += s_warp_sum[w];
    max_tiles = max(max_tiles, s_warp_max[w]);
  }
#pragma unroll
  for (int i = 0; i < kRowsPerThread; ++i) {
    const int b = threadIdx.x * rpt + i;
    if (i < rpt && b < batch) s_prefix[b] = excl * streams_per_row;
    excl += local[i];
  }
  total *= streams_per_row;
  if (threadIdx.x == 0) s_prefix[batch] = total;
  __syncthreads();

  // rows without a visible key have no tile: their zero outputs are dealt round-robin
  for (int b = blockIdx.x; b < batch; b += gridDim.x) {
    if (s_prefix[b + 1] != s_prefix[b]) continue;
    for (int sidx = 0; sidx < streams_per_row; ++sidx) {
      const int g0 = (sidx % group_tiles) * 8;
      fused_write_zero_row<T, D, kMmaThreads>(p.fused, b, (sidx / group_tiles) * p.groups + g0, min(8, p.groups - g0));
    }
  }
  if (total == 0) return;

  // tiles per CTA: an even share, at least one tile per warp, and long enough that no stream needs more partial slots
  // than the caller's scratch holds (a stream of n tiles touches at most ceil(n / tpc) + 1 CTAs)
  int tpc = (total + (int)gridDim.x - 1) / (int)gridDim.x;
  tpc = max(tpc, kBalancedMinTiles);
  tpc = max(tpc, (max_tiles + p.chunk_capacity - 2) / (p.chunk_capacity - 1));
  int pos = (int)min((int64_t)blockIdx.x * tpc, (int64_t)total);
  const int end = (int)min((int64_t)pos + tpc, (int64_t)total);
  if (pos >= end) return;

  // row that holds tile `pos`: the last b with s_prefix[b] <= pos (rows without tiles are skipped by construction)
  int lo = 0, hi = batch;  // invariant: s_prefix[lo] <= pos < s_prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_prefix[mid] <= pos) lo = mid; else hi = mid;
  }
  int b = lo;
  while (pos < end) {
    while (s_prefix[b + 1] <= pos) ++b;
    const int row_first = s_prefix[b];
    const int n = (s_prefix[b + 1] - row_first) / streams_per_row;  // tiles of each stream of this row
    const int sidx = (pos - row_first) / n;
    const int tile = (pos - row_first) - sidx * n;
    const int seg = min(n - tile, end - pos);
    const int stream_first = row_first + sidx * n;
    const int first_cta = stream_first / tpc;
    const int slot = (int)blockIdx.x - first_cta;
    const int active = (stream_first + n - 1) / tpc - first_cta + 1;
    const int kvh = sidx / group_tiles;
    const int g0 = (sidx % group_tiles) * 8;
    const int t0 = tile * kTileTokens;
    const int t1 = min(row_len(b), (tile + seg) * kTileTokens);
    dense_split_mma_body<T, D>(p, smem_raw, b, kvh, g0, min(8, p.groups - g0), t0, t1, slot, active,
                               (int64_t)b * streams_per_row + sidx);
    pos += seg;
    __syncthreads();  // the next segment reuses the pipeline and merge buffers
  }
}

template <typename T, int D>
static int launch_balanced(const DenseDecodeParams& p, int batch, cudaStream_t stream) {
  using Cfg = MmaCfg<D>;
  auto kernel = dense_decode_balanced_mma_kernel<T, D>;
  static int resident_ctas[64] = {};  // per device: CTAs of this kernel that fit the whole GPU at once
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  int ctas = (device >= 0 && device < 64) ? resident_ctas[device] : 0;
  if (ctas == 0) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    int sms = 0, per_sm = 0;
    ANNA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    ANNA_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kMmaThreads, Cfg::kSmemBytes));
    ctas = sms * (per_sm > 0 ? per_sm : 1);
    if (device >= 0 && device < 64) resident_ctas[device] = ctas;
  }
  kernel<<<(unsigned)ctas, kMmaThreads, Cfg::kSmemBytes, stream>>>(p, batch);
  return check_launch("dense_decode_balanced_mma_kernel");
}

bool dense_balanced_mma_applicable(const DenseDecodeParams& p, int batch) {
  static const bool disabled = [] {
    const char* flag = std::getenv("ANNA_B200_DISABLE_BALANCED");
    return flag != nullptr && flag[0] != '\0' && flag[0] != '0';
  }();
  if (disabled || p.fused.counters == nullptr) return false;
  if (batch > kBalancedMaxRows || p.chunk_capacity < 2) return false;
  const int64_t streams = (int64_t)batch * p.kv_heads * ((p.groups + 7) / 8);
  return streams * ((p.max_len + kTileTokens - 1) / kTileTokens) < ((int64_t)1 << 30);
}

int launch_dense_balanced_mma(const DenseDecodeParams& p, int batch, int head_dim, int dtype, cudaStream_t stream) {
  if (dtype == ANNA_DTYPE_BF16) {
    if (head_dim == 64) return launch_balanced<__nv_bfloat16, 64>(p, batch, stream);
    if (head_dim == 128) return launch_balanced<__nv_bfloat16, 128>(p, batch, stream);
    return launch_balanced<__nv_bfloat16, 256>(p, batch, stream);
  }
  if (head_dim == 64) return launch_balanced<__half, 64>(p, batch, stream);
  if (head_dim == 128) return launch_balanced<__half, 128>(p, batch, stream);
  return launch_balanced<__half, 256>(p, batch, stream);
}

template <typename T, int D>
static int launch_mma(const DenseDecodeParams& p, int batch, cudaStream_t stream) {
  using Cfg = MmaCfg<D>;
  auto kernel = dense_decode_split_mma_kernel<T, D>;
  static bool configured[64] = {};  // per device: the attribute belongs to the device's context
  int device = 0;
  ANNA_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= 64 || !configured[device]) {
    ANNA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  const int group_tiles = (p.groups + 7) / 8;
  dim3 grid((unsigned)p.num_chunks, (unsigned)(p.kv_heads * group_tiles), (unsigned)batch);
  kernel<<<grid, kMmaThreads, Cfg::kSmemBytes, stream>>>(p);
  return check_launch("dense_decode_split_mma_kernel");
}

bool dense_split_mma_applicable(const DenseDecodeParams& p, int head_dim, int dtype) {
  static const bool disabled = [] {
    const char* flag = std::getenv("ANNA_B200_DISABLE_MMA");
    return flag != nullptr && flag[0] != '\0' && flag[0] != '0';
  }();
  if (disabled) return false;
  if (dtype != ANNA_DTYPE_F16 && dtype != ANNA_DTYPE_BF16) return false;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return false;
  if (p.chunk_tokens % kTileTokens != 0 || p.max_len >= (int64_t)1 << 31) return false;
  // query rows are read as aligned 32-bit pairs
  if (p.q_stride_b % 2 != 0 || p.q_stride_h % 2 != 0 || (reinterpret_cast<uintptr_t>(p.q) & 3u) != 0) return false;
  return true;
}

int launch_dense_split_mma(const DenseDecodeParams& p, int batch, int head_dim, int dtype, cudaStream_t stream) {
  if (dtype == ANNA_DTYPE_BF16) {
    if (head_dim == 64) return launch_mma<__nv_bfloat16, 64>(p, batch, stream);
    if (head_dim == 128) return launch_mma<__nv_bfloat16, 128>(p, batch, stream);
    return launch_mma<__nv_bfloat16, 256>(p, batch, stream);
  }
  if (head_dim == 64) return launch_mma<__half, 64>(p, batch, stream);
  if (head_dim == 128) return launch_mma<__half, 128>(p, batch, stream);
  return launch_mma<__half, 256>(p, batch, stream);
}

}  // namespace anna
