#include "selftest_sm100.cuh"

#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

__global__ void __launch_bounds__(32) wait_timeout_kernel(uint32_t polls, uint32_t *status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ volatile uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    // Phase 0 never completes: nobody arrives.
    if (!mbar_wait_limited(&bar, 0, &abort_flag, polls)) {
      abort_flag = 1;
      atomicCAS(status, 0u, kStatusSelftestTimeout);
    }
  }
}

}  // namespace

cudaError_t selftest_wait_timeout(uint32_t polls, uint32_t *status, cudaStream_t stream) {
  wait_timeout_kernel<<<1, 32, 0, stream>>>(polls, status);
  return cudaGetLastError();
}

}  // namespace flsm100
