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
#include "balanced_schedule.cuh"
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
// Persistent variant: one resident wave, every CTA takes an even share of the tiles (balanced_schedule.cuh).
template <typename T, int D>
__global__ void __launch_bounds__(kMmaThreads, MmaCfg<D>::kMinBlocks)
dense_decode_balanced_mma_kernel(const DenseDecodeParams p, const int batch) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int group_tiles = (p.groups + 7) / 8;
  const int streams_per_row = p.kv_heads * group_tiles;
  // the fused merge stages at most kFusedMaxChunks weights per head, however large the caller's scratch is
  balanced_for_each_segment<kMmaThreads>(
      p.visible_lengths, p.max_len, batch, streams_per_row, min(p.chunk_capacity, kFusedMaxChunks),
      [&](int b) {
        for (int stream = 0; stream < streams_per_row; ++stream) {
          const int g0 = (stream % group_tiles) * 8;
          fused_write_zero_row<T, D, kMmaThreads>(p.fused, b, (stream / group_tiles) * p.groups + g0,
                                                  min(8, p.groups - g0));
        }
      },
      [&](int b, int stream, int t0, int t1, int slot, int partials) {
        const int g0 = (stream % group_tiles) * 8;
        dense_split_mma_body<T, D>(p, smem_raw, b, stream / group_tiles, g0, min(8, p.groups - g0), t0, t1, slot,
                                   partials, (int64_t)b * streams_per_row + stream);
        __syncthreads();  // the next segment reuses the pipeline and merge buffers
      });
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
  return balanced_schedule_fits(batch, (int64_t)p.kv_heads * ((p.groups + 7) / 8), p.max_len, p.chunk_capacity);
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
