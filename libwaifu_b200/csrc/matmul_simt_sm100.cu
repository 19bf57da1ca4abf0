#include "matmul_simt_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

namespace flsm100 {

namespace {

std::atomic<int64_t> g_launches{0};

constexpr int kTile = 64;    // rows and columns of out per CTA
constexpr int kStepK = 16;   // K positions staged per step
constexpr int kThreads = 256;  // 16 x 16 threads, 4 x 4 results each

template <int KIND>
__device__ __forceinline__ float load_as_float(const void *p, int64_t i) {
  if constexpr (KIND == kElemF32) {
    return reinterpret_cast<const float *>(p)[i];
  } else if constexpr (KIND == kElemBF16) {
    return __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t *>(p)[i]) << 16);
  } else {
    return __half2float(reinterpret_cast<const __half *>(p)[i]);
  }
}

template <int KIND>
__device__ __forceinline__ void store_from_float(void *p, int64_t i, float v) {
  if constexpr (KIND == kElemF32) {
    reinterpret_cast<float *>(p)[i] = v;
  } else if constexpr (KIND == kElemBF16) {
    reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
  } else {
    reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
  }
}

struct Params {
  const void *a, *b;
  void *out;
  int m, n, k;
  long long a_row, a_col, b_row, b_col;
  int batch_dims;
  int batch_shape[kMaxMatmulBatchDims];
  long long a_batch[kMaxMatmulBatchDims], b_batch[kMaxMatmulBatchDims];
  const void *bias, *residual;
  long long residual_rows, residual_ld;
};

// out[batch, i, j] = round(sum_k a[batch, i, k] b[batch, k, j] + bias[j] + residual[row % rows, j]).
// Each step stages 64 x 16 of a and 16 x 64 of b in shared memory as float32 through whatever strides
// the views have; a thread then takes 4 x 4 results through the staged K positions in order, so the
// sum of every result runs over k = 0, 1, 2, ... in one fp32 chain.
template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads) general_matmul_kernel(const Params p) {
  __shared__ float as[kStepK][kTile + 4];
  __shared__ float bs[kStepK][kTile + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * kTile, col0 = blockIdx.x * kTile;
  long long a_off = 0, b_off = 0;
  {
    int rest = blockIdx.z;
    for (int d = p.batch_dims - 1; d >= 0; --d) {
      const int idx = rest % p.batch_shape[d];
      rest /= p.batch_shape[d];
      a_off += idx * p.a_batch[d];
      b_off += idx * p.b_batch[d];
    }
  }
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.k; k0 += kStepK) {
    // 1024 elements of each operand per step, four per thread; consecutive threads walk the
    // dimension that is contiguous for a linear layer's operands (k for a, and for a transposed weight)
    for (int e = threadIdx.x; e < kTile * kStepK; e += kThreads) {
      const int kk = e % kStepK, r = e / kStepK;
      const int gr = row0 + r, gk = k0 + kk;
      as[kk][r] = (gr < p.m && gk < p.k) ? load_as_float<IN>(p.a, a_off + gr * p.a_row + gk * p.a_col) : 0.0f;
      const int gc = col0 + r;
      bs[kk][r] = (gc < p.n && gk < p.k) ? load_as_float<IN>(p.b, b_off + gk * p.b_row + gc * p.b_col) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kStepK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
    }
    __syncthreads();
  }
  const long long out_batch = static_cast<long long>(blockIdx.z) * p.m;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= p.m) continue;
    const long long global_row = out_batch + r;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= p.n) continue;
      float v = acc[i][j];
      if (p.bias) v += load_as_float<OUT>(p.bias, c);
      if (p.residual) v += load_as_float<OUT>(p.residual, (global_row % p.residual_rows) * p.residual_ld + c);
      store_from_float<OUT>(p.out, global_row * p.n + c, v);
    }
  }
}

}  // namespace

cudaError_t general_matmul(const GeneralMatmulArgs &a) {
  if (a.m <= 0 || a.n <= 0) return cudaSuccess;
  Params p = {};
  p.a = a.a, p.b = a.b, p.out = a.out;
  p.m = a.m, p.n = a.n, p.k = a.k;
  p.a_row = a.a_row, p.a_col = a.a_col, p.b_row = a.b_row, p.b_col = a.b_col;
  p.batch_dims = a.batch_dims;
  long long batches = 1;
  for (int d = 0; d < a.batch_dims; ++d) {
    p.batch_shape[d] = a.batch_shape[d];
    p.a_batch[d] = a.a_batch[d];
    p.b_batch[d] = a.b_batch[d];
    batches *= a.batch_shape[d];
  }
  if (batches <= 0) return cudaSuccess;
  if (batches > 65535) return cudaErrorInvalidValue;
  p.bias = a.bias, p.residual = a.residual;
  p.residual_rows = a.residual_rows > 0 ? a.residual_rows : 1;
  p.residual_ld = a.residual_ld;
  const dim3 grid((a.n + kTile - 1) / kTile, (a.m + kTile - 1) / kTile, static_cast<unsigned>(batches));
  if (grid.y > 65535) return cudaErrorInvalidValue;
#define FLSM100_LAUNCH(IN, OUT) general_matmul_kernel<IN, OUT><<<grid, kThreads, 0, a.stream>>>(p)
  if (a.in_kind == kElemF32 && a.out_kind == kElemF32) {
    FLSM100_LAUNCH(kElemF32, kElemF32);
  } else if (a.in_kind == kElemF16 && a.out_kind == kElemF16) {
    FLSM100_LAUNCH(kElemF16, kElemF16);
  } else if (a.in_kind == kElemF16 && a.out_kind == kElemF32) {
    FLSM100_LAUNCH(kElemF16, kElemF32);
  } else if (a.in_kind == kElemBF16 && a.out_kind == kElemBF16) {
    FLSM100_LAUNCH(kElemBF16, kElemBF16);
  } else if (a.in_kind == kElemBF16 && a.out_kind == kElemF32) {
    FLSM100_LAUNCH(kElemBF16, kElemF32);
  } else {
    return cudaErrorInvalidValue;
  }
#undef FLSM100_LAUNCH
  ++g_launches;
  return cudaGetLastError();
}

int64_t general_matmul_launch_count() { return g_launches.load(); }

}  // namespace flsm100
