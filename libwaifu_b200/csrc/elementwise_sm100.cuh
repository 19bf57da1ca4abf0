// The few elementwise operators a caller of the quantized-linear path needs around it
// (flint/capi.h:246-249,279,483): copy, cast, fill and add over views of float, half or bfloat16
// elements. All HBM-bound streaming kernels; none of them allocates.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

enum ElemKind : int { kElemF32 = 0, kElemF16 = 1, kElemBF16 = 2 };

constexpr int kMaxElemDims = 6;

// A view as the kernels see it: extents and element strides, innermost dimension last.
struct ElemView {
  const void *base;
  int ndim;
  int32_t shape[kMaxElemDims];
  int64_t stride[kMaxElemDims];
  bool contiguous;
};

// out[i] = convert(in[i]); out contiguous or strided, any pair of the three kinds (equal kinds: a copy).
cudaError_t elementwise_cast(const ElemView &in, ElemKind in_kind, const ElemView &out, ElemKind out_kind, int64_t numel,
                             cudaStream_t stream);
// view[i] = value, rounded to the view's kind once.
cudaError_t elementwise_fill(const ElemView &view, ElemKind kind, int64_t numel, float value, cudaStream_t stream);
// out[i] = round(a[i] + b[i]), the sum taken in fp32 (exact for 16-bit operands), one rounding.
cudaError_t elementwise_add(const ElemView &a, const ElemView &b, const ElemView &out, ElemKind kind, int64_t numel,
                            cudaStream_t stream);
// Byte-wise copy between views of `elem_bytes`-byte elements (1, 2, 4 or 8).
cudaError_t elementwise_copy(const ElemView &in, const ElemView &out, int elem_bytes, int64_t numel, cudaStream_t stream);

int64_t elementwise_launch_count();

}  // namespace flsm100
