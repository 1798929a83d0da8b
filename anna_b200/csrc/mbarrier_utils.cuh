// mbarrier and bulk-copy (TMA) primitives shared by the kernels that stage tiles with the copy engine.
//
// Protocol used everywhere: one mbarrier per ring stage, arrival count 1.  The lane that starts the copies of a tile
// arrives once with the expected byte count (or plainly, when there is nothing to copy); the copies complete the
// transaction count; consumers wait on the phase parity.  Every wait is bounded: after kWaitSpins suspended waits it
// gives up and reports false, so a kernel can never hang on a copy that does not arrive.
#pragma once

#include "mma_utils.cuh"

namespace anna {

constexpr uint32_t kWaitSpins = 1u << 16;      // bounded: at most this many suspended waits per tile
constexpr uint32_t kWaitHintNs = 20000u;       // a waiting warp sleeps in hardware instead of polling

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
// Makes freshly initialised barriers visible to the copy engine; follow it with a CTA barrier.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kWaitSpins; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    if (done) return true;
  }
  return false;
}
// Linear copy of `bytes` (a multiple of 16) from global `src` to shared `dst`, both 16-byte aligned; the bytes are
// counted on `bar` as they land.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

}  // namespace anna
