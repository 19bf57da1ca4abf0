#include "peer_sm100.cuh"

namespace flsm100 {

namespace {

constexpr int kThreads = 1024;

struct Boxes {
  int32_t *at[kPeerMaxRanks];
};

__device__ __forceinline__ void store_release_system(int32_t *p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int32_t load_acquire_system(const int32_t *p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreads) peer_exchange_kernel(Boxes boxes, int n_ranks, int rank, int64_t ld, int32_t epoch,
                                                                 float *row_amax, int rows, uint32_t max_polls,
                                                                 uint32_t *status) {
  __shared__ int gave_up;
  const int tid = threadIdx.x;
  if (tid == 0) gave_up = 0;
  if (row_amax) {
    for (int p = 0; p < n_ranks; ++p) {
      int32_t *payload = boxes.at[p] + rank * ld + kPeerHeaderWords;
      for (int i = tid; i < rows; i += kThreads) payload[i] = __float_as_int(row_amax[i]);
    }
  }
  __syncthreads();
  if (tid < n_ranks) {
    // the fence is cumulative: the payload above (ordered by the barrier) and what earlier kernels of
    // this stream wrote into peers' memory become visible before the flag does
    __threadfence_system();
    store_release_system(boxes.at[tid] + rank * ld, epoch);
    const int32_t *flag = boxes.at[rank] + tid * ld;
    bool seen = false;
    for (uint32_t poll = 0; poll < max_polls; ++poll) {
      if (load_acquire_system(flag) - epoch >= 0) {
        seen = true;
        break;
      }
      __nanosleep(200);
    }
    if (!seen) {
      gave_up = 1;
      atomicCAS(status, 0u, kStatusPeerTimeout);
    }
  }
  __syncthreads();
  if (gave_up || !row_amax) return;
  const int32_t *mine = boxes.at[rank];
  for (int i = tid; i < rows; i += kThreads) {
    int32_t v = 0;
    for (int p = 0; p < n_ranks; ++p) v = max(v, __ldcg(mine + p * ld + kPeerHeaderWords + i));  // past L1: peers wrote these
    row_amax[i] = __int_as_float(v);
  }
}

}  // namespace

cudaError_t peer_exchange(const PeerExchangeArgs &a) {
  Boxes boxes;
  for (int i = 0; i < kPeerMaxRanks; ++i) boxes.at[i] = i < a.n_ranks ? a.mailbox[i] : nullptr;
  peer_exchange_kernel<<<1, kThreads, 0, a.stream>>>(boxes, a.n_ranks, a.rank, a.ld, a.epoch, a.row_amax, a.rows,
                                                     a.max_polls ? a.max_polls : kPeerDefaultPolls, a.status);
  return cudaGetLastError();
}

}  // namespace flsm100
