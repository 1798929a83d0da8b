// Tiled TMA loads (cp.async.bulk.tensor) and the host-side tensor-map encoder, looked up at run time so that nothing
// links against libcuda.  Coordinates: the innermost one times the element size must be a multiple of 16 bytes; loads
// may start past the tensor's extent and read zeros there.  Every load is addressed to the issuing CTA alone.
#pragma once

#include <cuda.h>  // CUtensorMap and its enums

#include "common.cuh"

namespace anna {

// One 2-D box: elements [x, x + box_x) of rows [y, y + box_y) -> shared `dst`, completion bytes counted on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// One 4-D box (x innermost).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, int w, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n" ::
          "r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
      : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Tensor map of a 16-bit tensor of `rank` dimensions (extents and byte strides innermost first; strides[0] is the
// stride of dimension 1), 128-byte swizzle, zeros outside.  False when the encoder is missing or refuses.
inline bool encode_map_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* extents,
                             const uint64_t* byte_strides, const uint32_t* box) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr || rank < 1 || rank > 5) return false;
  cuuint64_t dims[5], strides[4];
  cuuint32_t boxes[5], elem[5];
  for (int i = 0; i < rank; ++i) {
    dims[i] = extents[i];
    boxes[i] = box[i];
    elem[i] = 1;
    if (i + 1 < rank) strides[i] = byte_strides[i];
  }
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, boxes, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace anna
