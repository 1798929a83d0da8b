// Arrival flags between the GPUs of one box for the KV-head-sharded decode.
//
// Every rank owns an array of `world` 64-bit flags in memory its peers can write (flag r is written by rank r only).
// After a decode whose merge stored this rank's output rows into the peers' output tensors, one warp publishes the step
// number into flag `rank` of every peer (release at system scope, so the rows are visible before the number is) and
// then waits until its own flags show that every peer has published the same step.  The wait is bounded: when the budget
// runs out the kernel ORs ANNA_DEV_PEER_TIMEOUT into the status word and returns, and the context stays usable.
// Steps only grow, so a flag is never reset and a late reader cannot miss a value.
#include "common.cuh"

namespace anna {

struct PeerFlags {
  unsigned long long* arrays[kMaxPeerOutputs + 1];  // flag array of every rank; arrays[rank] is this rank's own
  int rank, world;
  unsigned long long step;
  long long budget_ns;
  int32_t* status;
};

__device__ __forceinline__ void st_release_sys(unsigned long long* ptr, unsigned long long value) {
  asm volatile("st.release.sys.global.u64 [%0], %1;\n" ::"l"(ptr), "l"(value) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* ptr) {
  unsigned long long value;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];\n" : "=l"(value) : "l"(ptr) : "memory");
  return value;
}
__device__ __forceinline__ long long global_timer_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(32) peer_signal_wait_kernel(const PeerFlags f) {
  const int peer = threadIdx.x;
  if (peer >= f.world || peer == f.rank) return;
  st_release_sys(f.arrays[peer] + f.rank, f.step);
  const unsigned long long* mine = f.arrays[f.rank] + peer;
  const long long start = global_timer_ns();
  while (ld_acquire_sys(mine) < f.step) {
    if (global_timer_ns() - start > f.budget_ns) {
      if (f.status != nullptr) atomicOr(f.status, (int)ANNA_DEV_PEER_TIMEOUT);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace anna

using namespace anna;

extern "C" int anna_peer_signal_wait(void* const* flag_arrays, int rank, int world, int64_t step, int64_t timeout_ms,
                                     int32_t* status, anna_stream_t stream) {
  ANNA_REQUIRE(flag_arrays != nullptr, "anna_peer_signal_wait: null flag array table");
  ANNA_REQUIRE(world >= 1 && world <= kMaxPeerOutputs + 1 && rank >= 0 && rank < world,
               "anna_peer_signal_wait: rank %d of %d (at most %d ranks)", rank, world, kMaxPeerOutputs + 1);
  ANNA_REQUIRE(step > 0, "anna_peer_signal_wait: steps are positive and grow from call to call");
  ANNA_REQUIRE(timeout_ms > 0 && timeout_ms <= 60000, "anna_peer_signal_wait: timeout must be within (0, 60000] ms");
  PeerFlags f{};
  for (int r = 0; r < world; ++r) {
    ANNA_REQUIRE(flag_arrays[r] != nullptr && (reinterpret_cast<uintptr_t>(flag_arrays[r]) & 7u) == 0,
                 "anna_peer_signal_wait: flag array %d is null or not 8-byte aligned", r);
    f.arrays[r] = reinterpret_cast<unsigned long long*>(flag_arrays[r]);
  }
  f.rank = rank; f.world = world; f.step = (unsigned long long)step; f.budget_ns = timeout_ms * 1000000ll; f.status = status;
  if (world == 1) return ANNA_OK;
  peer_signal_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f);
  return check_launch("peer_signal_wait_kernel");
}
