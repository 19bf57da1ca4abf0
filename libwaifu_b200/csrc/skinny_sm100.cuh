// The bandwidth-shaped FP8 linear for at most 16 activation rows (see skinny_sm100.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

// Whether the skinny kernel takes this shape: 1..16 rows, n a multiple of 8, k of 16, a 16-byte
// aligned weight, and activation rows (and residual rows, if any) that leave shared memory for at
// least three ring stages.
// `status` in the calls below is the device-visible word a bounded wait that gave up reports to.
bool skinny_fp8_supported(int m, int n, int k, const void *x, const void *w, const void *out, bool has_residual);

// out = round16( act( (x_q . w) * (row scale * channel scale) + bias ) + residual ), with x
// quantised per row inside the kernel exactly as quantize_fp8_act does. One launch, no scratch.
cudaError_t skinny_fp8_linear(const void *x, int is_bf16, int m, int n, int k, const uint8_t *w, const float *col_scale,
                              int col_scale_scalar, const void *bias, const void *residual, int act, void *out,
                              uint32_t *status, cudaStream_t stream);

// The reference-compatible product for at most 16 rows: the activation is not narrowed, the e4m3
// weight is widened to the activation's 16-bit type in registers, one <float> scale, an optional
// bias (n) and/or residual rows (period residual_rows over m, pitch residual_ld) added to the fp32
// sum, one rounding (flint/cuda/gemm_fp8_cutlass.cu:107-125).
bool skinny_upcast_supported(int m, int n, int k, const void *x, const void *w, const void *out, bool has_residual);
cudaError_t skinny_upcast_matmul(const void *x, int is_bf16, int m, int n, int k, const uint8_t *w, const float *scale,
                                 const void *bias, const void *residual, int residual_rows, int64_t residual_ld,
                                 void *out, uint32_t *status, cudaStream_t stream);

// The unquantised linear layer for at most 16 rows: x (m, k) times the transpose of a 16-bit
// weight (n, k) of the same type, fp32 accumulation, an optional bias (n) and/or residual rows
// added to the fp32 sum, one rounding (the GEMV of flint/cuda/matvec.cu and the bias-in-epilogue
// of flint/cuda/gemm_cutlass.cu:208-235 in one kernel).
bool skinny_w16_supported(int m, int n, int k, const void *x, const void *w, const void *out, bool has_residual);
cudaError_t skinny_w16_matmul(const void *x, int is_bf16, int m, int n, int k, const void *w, const void *bias,
                              const void *residual, int residual_rows, int64_t residual_ld, void *out,
                              uint32_t *status, cudaStream_t stream);

// The shared-memory and K-split plan the kernel would run a shape with (host arithmetic only, for
// checks that need no GPU): 16 values, see fl_sm100_few_rows_plan. Returns 0 when the shape is
// not taken.
int skinny_plan(int m, int n, int k, int wbytes, int xbytes, int has_residual, int32_t *out);

}  // namespace flsm100
