// Bounded counting wait kernel (see fo_wait.h).
#include "fo_wait.h"

#include "../common/fo_ptx.cuh"

namespace fo {

namespace {

__global__ void wait_flag_kernel(int target, int* addr, int group, uint64_t timeout_ns,
                                 int32_t* status) {
  const uint64_t t0 = ptx::cycles_now();
  const uint64_t budget = ptx::ns_to_cycles(timeout_ns);
  uint32_t it = 0;
  int seen = 0;
  while (true) {
    // Succeeds exactly when the counter equals the group's tile count; the swap to 0 re-arms
    // the counter for the next call without a separate memset.
    seen = atomicCAS(addr, target, 0);
    if (seen == target) {
      __threadfence();  // acquire side: later work on this stream sees the tiles
      return;
    }
    __nanosleep(100);
    if ((++it & 63u) == 0u && ptx::cycles_now() - t0 > budget) break;
  }
  ptx::report_status(status, kStatusTimeoutWaitKernel, group, seen, target);
}

}  // namespace

cudaError_t wait_flag_launch(int target, int* addr, int group, uint64_t timeout_ns, int32_t* status,
                             cudaStream_t stream) {
  wait_flag_kernel<<<1, 1, 0, stream>>>(target, addr, group, timeout_ns, status);
  return cudaGetLastError();
}

}  // namespace fo
