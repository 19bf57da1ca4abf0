// The general matrix product behind fl_matmul / fl_matmul_add for every operand layout the tensor-core
// kernel does not take: float32 operands, a float32 result from 16-bit operands, batches on either
// operand, a right operand that is not a transposed linear-layer weight, extents that are not
// multiples of 8 (flint/cuda/matmul.cc:315-343 serves these through cuBLAS or CUTLASS kernels). A
// plain tiled kernel on the FP32 pipes with fp32 accumulation: these products are the small ones of
// a model (a 129-channel input projection, the composed attention of a test), and what matters for
// them is that they are served at all and rounded once.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "elementwise_sm100.cuh"

namespace flsm100 {

constexpr int kMaxMatmulBatchDims = 4;

struct GeneralMatmulArgs {
  const void *a, *b;
  void *out;
  ElemKind in_kind, out_kind;   // operands of one kind; the result of the same kind, or float32
  int m, n, k;
  int64_t a_row, a_col;         // element strides of a's last two dimensions (m, k)
  int64_t b_row, b_col;         // of b's last two dimensions (k, n)
  int batch_dims;               // leading dimensions, outermost first
  int32_t batch_shape[kMaxMatmulBatchDims];
  int64_t a_batch[kMaxMatmulBatchDims], b_batch[kMaxMatmulBatchDims];  // 0 where the operand is broadcast
  // out is contiguous (batches..., m, n). Added to the fp32 sum before the one rounding:
  const void *bias;             // (n) of the result's kind, or null
  const void *residual;         // rows of n of the result's kind repeating with a period over all rows of out, or null
  int64_t residual_rows, residual_ld;
  cudaStream_t stream;
};

cudaError_t general_matmul(const GeneralMatmulArgs &args);
int64_t general_matmul_launch_count();

}  // namespace flsm100
