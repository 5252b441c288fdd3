// Counting wait kernel for the counter-gated NCCL path.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace fo {

// Enqueues a 1-thread kernel on `stream` that returns once *addr == target, resetting the
// counter to 0 in the same atomic, as the reference's kernel_wait_flag does
// (src/wait.cuh:5-9).  Unlike the reference the wait is bounded: after `timeout_ns` the
// kernel writes kStatusTimeoutWaitKernel (with the group index, the observed and the
// expected count) to `status` and returns, so a missing signal never hangs the GPU.
cudaError_t wait_flag_launch(int target, int* addr, int group, uint64_t timeout_ns, int32_t* status,
                             cudaStream_t stream);

}  // namespace fo
