// Self-test of the tensor-memory matrix-multiply primitives (umma_utils.cuh) in the two operand arrangements the packed
// decode uses:
//   D1[128 x 16] = A1[128 x 128] . B1[16 x 128]^T    e4m3 operands, both K-major          (scores: tokens x heads)
//   D2[128 x 16] = A2[128 x 128]^T . B2[128 x 16]    f16 operands, both MN-major          (values: dims x heads)
// Operands arrive as plain row-major device arrays, the kernel re-tiles them into the canonical shared-memory layouts
// with the padded strides of the real kernel, multiplies, and returns the accumulators.  No counterpart in the reference.
#include "tma_utils.cuh"
#include "umma_utils.cuh"

namespace anna {

constexpr int kSelfM = 128, kSelfN = 16, kSelfK = 128;
// strides of the canonical layouts (bytes); the odd multiples of 16 spread a warp's 16-byte stores over all banks
constexpr uint32_t kA1Sbo = 128, kA1Lbo = 128 * 16 + 16;   // K-major A: 8-row groups back to back, K chunks padded
constexpr uint32_t kB1Sbo = 128, kB1Lbo = 256;             // K-major B: 16 rows = two groups per K chunk
constexpr uint32_t kA2Sbo = 144, kA2Lbo = 16 * 144;        // MN-major A: 16 groups of 8 rows per 8 K indices, padded
constexpr uint32_t kB2Sbo = 128, kB2Lbo = 256;             // MN-major B: two groups of 8 columns per 8 K indices
constexpr uint32_t kA1Bytes = 8 * kA1Lbo, kB1Bytes = 8 * kB1Lbo, kA2Bytes = 16 * kA2Lbo, kB2Bytes = 16 * kB2Lbo;
constexpr uint32_t kSelfSmem = kA1Bytes + kB1Bytes + kA2Bytes + kB2Bytes;

__global__ void __launch_bounds__(128) umma_selftest_kernel(const uint8_t* a1, const uint8_t* b1, const __half* a2,
                                                            const __half* b2, float* d1, float* d2, int32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ uint32_t tmem_slot;
  uint8_t* s_a1 = smem;
  uint8_t* s_b1 = s_a1 + kA1Bytes;
  uint8_t* s_a2 = s_b1 + kB1Bytes;
  uint8_t* s_b2 = s_a2 + kA2Bytes;
  const uint32_t bar = smem_u32(&bar_storage);
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 32);
  // re-tile the operands
  for (int i = threadIdx.x; i < kSelfM * kSelfK; i += blockDim.x) {  // A1[r][k], one byte each
    const int r = i / kSelfK, k = i % kSelfK;
    s_a1[(r / 8) * kA1Sbo + (k / 16) * kA1Lbo + (r % 8) * 16 + k % 16] = a1[i];
  }
  for (int i = threadIdx.x; i < kSelfN * kSelfK; i += blockDim.x) {  // B1[n][k]
    const int r = i / kSelfK, k = i % kSelfK;
    s_b1[(r / 8) * kB1Sbo + (k / 16) * kB1Lbo + (r % 8) * 16 + k % 16] = b1[i];
  }
  for (int i = threadIdx.x; i < kSelfK * kSelfM; i += blockDim.x) {  // A2[k][m]: K index k, row m (2 bytes each)
    const int k = i / kSelfM, m = i % kSelfM;
    *reinterpret_cast<__half*>(s_a2 + (m / 8) * kA2Sbo + (k / 8) * kA2Lbo + (k % 8) * 16 + (m % 8) * 2) = a2[i];
  }
  for (int i = threadIdx.x; i < kSelfK * kSelfN; i += blockDim.x) {  // B2[k][n]
    const int k = i / kSelfN, n = i % kSelfN;
    *reinterpret_cast<__half*>(s_b2 + (n / 8) * kB2Sbo + (k / 8) * kB2Lbo + (k % 8) * 16 + (n % 8) * 2) = b2[i];
  }
  fence_async_smem();
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc1 = umma_idesc(kUmmaE4M3, kUmmaE4M3, false, false, kSelfM, kSelfN);
    constexpr uint32_t idesc2 = umma_idesc(kUmmaF16, kUmmaF16, true, true, kSelfM, kSelfN);
    for (int k = 0; k < kSelfK / 32; ++k)  // 32 e4m3 values of K per instruction = two 16-byte chunks
      umma_f8(tmem, umma_smem_desc(smem_u32(s_a1) + 2 * k * kA1Lbo, kA1Lbo, kA1Sbo),
              umma_smem_desc(smem_u32(s_b1) + 2 * k * kB1Lbo, kB1Lbo, kB1Sbo), idesc1, k > 0);
    for (int k = 0; k < kSelfK / 16; ++k)  // 16 f16 values of K per instruction = two groups of 8 K indices
      umma_f16(tmem + 16, umma_smem_desc(smem_u32(s_a2) + 2 * k * kA2Lbo, kA2Lbo, kA2Sbo),
               umma_smem_desc(smem_u32(s_b2) + 2 * k * kB2Lbo, kB2Lbo, kB2Sbo), idesc2, k > 0);
    umma_commit(bar);
  }
  const bool landed = mbar_wait(bar, 0u);
  tcgen05_fence_after_sync();
  if (landed) {
    uint32_t r1[16], r2[16];
    tmem_ld16(tmem_addr(tmem, 32 * warp, 0), r1);
    tmem_ld16(tmem_addr(tmem, 32 * warp, 16), r2);
    tmem_wait_ld();
    for (int j = 0; j < 16; ++j) {
      d1[threadIdx.x * 16 + j] = __uint_as_float(r1[j]);
      d2[threadIdx.x * 16 + j] = __uint_as_float(r2[j]);
    }
  } else if (threadIdx.x == 0) {
    *status = 1;  // the multiply never reported completion
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 32);
}

// Second self-test: operands brought in by tiled TMA loads with the 128-byte swizzle and read through swizzled
// descriptors, in the two arrangements of the tensor-memory prefill kernel:
//   D1[128 x 128] = A[128 x 128] . B1[128 x 128]^T     bf16, A and B1 K-major (rows of A / B1 are rows of the tensors)
//   D2[128 x 128] = A[128 x 128] . B2[128 x 128]       bf16, B2 MN-major (its rows are K indices, as V's rows are keys)
constexpr uint32_t kTmaBox = 128 * 128;   // bytes of one box: 128 rows x 64 values
__global__ void __launch_bounds__(128) umma_tma_selftest_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_b1,
                                                                const __grid_constant__ CUtensorMap map_b2, float* d1,
                                                                float* d2, int32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) unsigned long long bar_storage[2];
  __shared__ uint32_t tmem_slot;
  const uint32_t base = (smem_u32(smem) + 1023u) & ~1023u;
  const uint32_t s_a = base, s_b1 = base + 2 * kTmaBox, s_b2 = base + 4 * kTmaBox;
  const uint32_t bar_load = smem_u32(&bar_storage[0]), bar_mma = smem_u32(&bar_storage[1]);
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 256);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    mbar_expect_tx(bar_load, 6 * kTmaBox);
    for (int h = 0; h < 2; ++h) {  // columns [64h, 64h + 64) of all 128 rows
      tma_load_2d(s_a + h * kTmaBox, &map_a, 64 * h, 0, bar_load);
      tma_load_2d(s_b1 + h * kTmaBox, &map_b1, 64 * h, 0, bar_load);
      tma_load_2d(s_b2 + h * kTmaBox, &map_b2, 64 * h, 0, bar_load);
    }
  }
  bool ok = __syncthreads_and(mbar_wait(bar_load, 0u));
  if (ok && threadIdx.x == 0) {
    tcgen05_fence_after_sync();
    constexpr uint32_t idesc1 = umma_idesc(kUmmaBF16, kUmmaBF16, false, false, 128, 128);
    constexpr uint32_t idesc2 = umma_idesc(kUmmaBF16, kUmmaBF16, false, true, 128, 128);
    for (int k = 0; k < 8; ++k) {  // 16 values of K per instruction: 32 bytes inside a 128-byte row, 4 per box
      const uint32_t off = (k / 4) * kTmaBox + (k % 4) * 32;
      umma_f16(tmem, umma_smem_desc_sw128(s_a + off, 16, 1024), umma_smem_desc_sw128(s_b1 + off, 16, 1024), idesc1, k > 0);
    }
    for (int k = 0; k < 8; ++k) {  // 16 K indices = 16 rows of B2 = 2048 bytes; the second 64 columns are the next box
      const uint32_t off = (k / 4) * kTmaBox + (k % 4) * 32;
      umma_f16(tmem + 128, umma_smem_desc_sw128(s_a + off, 16, 1024),
               umma_smem_desc_sw128(s_b2 + k * 2048, kTmaBox, 1024), idesc2, k > 0);
    }
    umma_commit(bar_mma);
  }
  if (ok) ok = __syncthreads_and(mbar_wait(bar_mma, 0u));
  tcgen05_fence_after_sync();
  if (ok) {
    for (int c = 0; c < 16; ++c) {
      uint32_t r[16];
      tmem_ld16(tmem_addr(tmem, 32 * warp, 16 * c), r);
      tmem_wait_ld();
      for (int j = 0; j < 16; ++j) {
        if (c < 8) d1[threadIdx.x * 128 + 16 * c + j] = __uint_as_float(r[j]);
        else d2[threadIdx.x * 128 + 16 * (c - 8) + j] = __uint_as_float(r[j]);
      }
    }
  } else if (threadIdx.x == 0) {
    *status = 1;
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

// Third self-test: the A operand in tensor memory (the P . V arrangement of the prefill kernel once P stays there):
//   D[128 x 128] = A[128 x 128] . B[128 x 128]     bf16; thread r packs row r of A into 64 columns of its lane with
//                                                  tcgen05.st, B arrives by TMA, MN-major
__global__ void __launch_bounds__(128) umma_ts_selftest_kernel(const __nv_bfloat16* a, const __grid_constant__ CUtensorMap map_b,
                                                               float* d, int32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) unsigned long long bar_storage[2];
  __shared__ uint32_t tmem_slot;
  const uint32_t s_b = (smem_u32(smem) + 1023u) & ~1023u;
  const uint32_t bar_load = smem_u32(&bar_storage[0]), bar_mma = smem_u32(&bar_storage[1]);
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 256);
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    mbar_expect_tx(bar_load, 2 * kTmaBox);
    for (int h = 0; h < 2; ++h) tma_load_2d(s_b + h * kTmaBox, &map_b, 64 * h, 0, bar_load);
  }
  // row threadIdx.x of A: 128 values = 64 columns (two per column, the lower K index in the lower half)
  const uint32_t* a_row = reinterpret_cast<const uint32_t*>(a + threadIdx.x * 128);
  for (int c = 0; c < 4; ++c) {
    uint32_t r[16];
    for (int j = 0; j < 16; ++j) r[j] = a_row[16 * c + j];
    tmem_st16(tmem_addr(tmem, 32 * warp, 16 * c), r);
  }
  tmem_wait_st();
  tcgen05_fence_before_sync();
  bool ok = __syncthreads_and(mbar_wait(bar_load, 0u));
  if (ok && threadIdx.x == 0) {
    tcgen05_fence_after_sync();
    constexpr uint32_t idesc = umma_idesc(kUmmaBF16, kUmmaBF16, false, true, 128, 128);
    for (int k = 0; k < 8; ++k)  // 16 K indices: eight columns of A, 16 rows of B = 2048 bytes
      umma_f16_ts(tmem + 128, tmem + 8 * k, umma_smem_desc_sw128(s_b + k * 2048, kTmaBox, 1024), idesc, k > 0);
    umma_commit(bar_mma);
  }
  if (ok) ok = __syncthreads_and(mbar_wait(bar_mma, 0u));
  tcgen05_fence_after_sync();
  if (ok) {
    for (int c = 0; c < 8; ++c) {
      uint32_t r[16];
      tmem_ld16(tmem_addr(tmem, 32 * warp, 128 + 16 * c), r);
      tmem_wait_ld();
      for (int j = 0; j < 16; ++j) d[threadIdx.x * 128 + 16 * c + j] = __uint_as_float(r[j]);
    }
  } else if (threadIdx.x == 0) {
    *status = 1;
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_free(tmem, 256);
}

}  // namespace anna

// a1 uint8 [128][128] (e4m3 bytes), b1 uint8 [16][128], a2 f16 [128 (K)][128 (rows)], b2 f16 [128 (K)][16]:
// d1 float [128][16] = a1 . b1^T, d2 float [128][16] = a2^T . b2.  *status = 1 when the tensor core did not report back
// within the bounded wait.  Synchronises the stream.
extern "C" int anna_kv_selftest_umma(const void* a1, const void* b1, const void* a2, const void* b2, float* d1,
                                     float* d2, int* status, anna_stream_t stream) {
  using namespace anna;
  ANNA_REQUIRE(a1 && b1 && a2 && b2 && d1 && d2 && status, "anna_kv_selftest_umma: null pointer argument");
  int32_t* flag = nullptr;
  ANNA_CUDA_CHECK(cudaMalloc(&flag, sizeof(int32_t)));
  cudaError_t err = cudaMemsetAsync(flag, 0, sizeof(int32_t), (cudaStream_t)stream);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSelfSmem);
  if (err == cudaSuccess) {
    umma_selftest_kernel<<<1, 128, kSelfSmem, (cudaStream_t)stream>>>(
        static_cast<const uint8_t*>(a1), static_cast<const uint8_t*>(b1), static_cast<const __half*>(a2),
        static_cast<const __half*>(b2), d1, d2, flag);
    err = cudaGetLastError();
  }
  int32_t value = -1;
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(&value, flag, sizeof(value), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize((cudaStream_t)stream);
  cudaFree(flag);
  if (err != cudaSuccess) return set_error(ANNA_ERR_CUDA, "tensor-memory self-test failed: %s", cudaGetErrorString(err));
  *status = (int)value;
  return ANNA_OK;
}

// a, b1, b2: bf16 [128][128] row-major device arrays (16-byte aligned); d1 = a . b1^T, d2 = a . b2 (float [128][128]).
// The operands travel by tiled TMA loads with the 128-byte swizzle.  *status = 1 when a bounded wait ran out, 2 when the
// driver's tensor-map encoder is not available.  Synchronises the stream.  No counterpart in the reference.
extern "C" int anna_kv_selftest_umma_tma(const void* a, const void* b1, const void* b2, float* d1, float* d2, int* status,
                                         anna_stream_t stream) {
  using namespace anna;
  ANNA_REQUIRE(a && b1 && b2 && d1 && d2 && status, "anna_kv_selftest_umma_tma: null pointer argument");
  CUtensorMap maps[3];
  const void* bases[3] = {a, b1, b2};
  const uint64_t extents[2] = {128, 128};
  const uint64_t strides[1] = {256};
  const uint32_t box[2] = {64, 128};
  for (int i = 0; i < 3; ++i)
    if (!encode_map_16bit(&maps[i], bases[i], 2, extents, strides, box)) {
      *status = 2;
      return ANNA_OK;
    }
  int32_t* flag = nullptr;
  ANNA_CUDA_CHECK(cudaMalloc(&flag, sizeof(int32_t)));
  constexpr int kSmem = 6 * (int)kTmaBox + 1024;
  cudaError_t err = cudaMemsetAsync(flag, 0, sizeof(int32_t), (cudaStream_t)stream);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(umma_tma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (err == cudaSuccess) {
    umma_tma_selftest_kernel<<<1, 128, kSmem, (cudaStream_t)stream>>>(maps[0], maps[1], maps[2], d1, d2, flag);
    err = cudaGetLastError();
  }
  int32_t value = -1;
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(&value, flag, sizeof(value), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize((cudaStream_t)stream);
  cudaFree(flag);
  if (err != cudaSuccess)
    return set_error(ANNA_ERR_CUDA, "tensor-memory / TMA self-test failed: %s", cudaGetErrorString(err));
  *status = (int)value;
  return ANNA_OK;
}

// a, b: bf16 [128][128] row-major device arrays (16-byte aligned); d = a . b (float [128][128]) with a held in tensor
// memory and b brought in by TMA.  *status as for anna_kv_selftest_umma_tma.  Synchronises the stream.  No counterpart in
// the reference.
extern "C" int anna_kv_selftest_umma_ts(const void* a, const void* b, float* d, int* status, anna_stream_t stream) {
  using namespace anna;
  ANNA_REQUIRE(a && b && d && status, "anna_kv_selftest_umma_ts: null pointer argument");
  CUtensorMap map;
  const uint64_t extents[2] = {128, 128};
  const uint64_t strides[1] = {256};
  const uint32_t box[2] = {64, 128};
  if (!encode_map_16bit(&map, b, 2, extents, strides, box)) {
    *status = 2;
    return ANNA_OK;
  }
  int32_t* flag = nullptr;
  ANNA_CUDA_CHECK(cudaMalloc(&flag, sizeof(int32_t)));
  constexpr int kSmem = 2 * (int)kTmaBox + 1024;
  cudaError_t err = cudaMemsetAsync(flag, 0, sizeof(int32_t), (cudaStream_t)stream);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(umma_ts_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (err == cudaSuccess) {
    umma_ts_selftest_kernel<<<1, 128, kSmem, (cudaStream_t)stream>>>(static_cast<const __nv_bfloat16*>(a), map, d, flag);
    err = cudaGetLastError();
  }
  int32_t value = -1;
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(&value, flag, sizeof(value), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize((cudaStream_t)stream);
  cudaFree(flag);
  if (err != cudaSuccess)
    return set_error(ANNA_ERR_CUDA, "tensor-memory operand self-test failed: %s", cudaGetErrorString(err));
  *status = (int)value;
  return ANNA_OK;
}
