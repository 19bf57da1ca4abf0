// A self-test of the bounded-wait machinery every kernel of this library relies on.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

// Status code the self-test kernel reports when its wait ran out (which is what it is for).
constexpr uint32_t kStatusSelftestTimeout = 0x51;

// One warp initialises an mbarrier that nothing ever arrives on and waits for it with a limit of
// `polls` try_wait polls. No TMA, no tensor memory, nothing in flight: when the limit is reached
// the kernel writes kStatusSelftestTimeout into *status (if it is still 0) and returns normally,
// exactly as the GEMM and attention kernels do when one of their waits gives up.
cudaError_t selftest_wait_timeout(uint32_t polls, uint32_t *status, cudaStream_t stream);

}  // namespace flsm100
