// The reference-compatible product for at most 16 half rows on tensor cores: the weight on the M
// side of tcgen05.mma, widened from shared memory into tensor memory, the rows as N = 16 (see
// fewrow_tc_sm100.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

constexpr uint32_t kStatusFewRowTcTimeout = 0x71;

// 1..64 half rows (not bfloat16: the widened weight and the rows have to be one type), k a
// multiple of 64, n a multiple of 8, x and w 16-byte aligned.
bool fewrow_tc_supported(int m, int n, int k, int is_bf16, const void *x, const void *w, const void *out);

// out (m, n) = round16( (x . widen(w)^T) * scale + bias (n) + residual rows (period residual_rows over
// m, pitch residual_ld) ), x (m, k) half, w (n, k) e4m3, one <float> scale, fp32 accumulation
// (flint/cuda/gemm_fp8_cutlass.cu:107-125). One launch, no scratch.
cudaError_t fewrow_tc_matmul(const void *x, int m, int n, int k, const uint8_t *w, const float *scale, const void *bias,
                             const void *residual, int residual_rows, int64_t residual_ld, void *out, uint32_t *status,
                             cudaStream_t stream, const char **why);

// e4m3 rows (a quantiser's codes, one <float> scale per row) against an e4m3 weight, for at most
// 64 rows: k a multiple of 16, n a multiple of 8, codes and w 16-byte aligned.
bool fewrow_q8_supported(int m, int n, int k, const void *codes, const void *w, const void *out);

// out (m, n) = round16( act( (codes . w^T) * (row_scale[row] * col_scale[channel or 0]) + bias ) + residual ),
// the arithmetic of fl_fp8_linear's epilogue in its order (fp32 accumulation). One launch, no scratch.
cudaError_t fewrow_q8_linear(const uint8_t *codes, const float *row_scale, int m, int n, int k, const uint8_t *w,
                             const float *col_scale, int col_scale_scalar, const void *bias, const void *residual,
                             int residual_rows, int64_t residual_ld, int act, int is_bf16, void *out, uint32_t *status,
                             cudaStream_t stream, const char **why);

// The same kernel on 16-bit operands (fl_matmul's linear-layer case, kind::f16): x (m, k) and w (n, k)
// half or bfloat16, out = round16(x . w^T + bias (n) + residual rows). At most 64 rows, k and n
// multiples of 8, x and w 16-byte aligned.
bool fewrow_w16_supported(int m, int n, int k, const void *x, const void *w, const void *out);
cudaError_t fewrow_w16_matmul(const void *x, int is_bf16, int m, int n, int k, const void *w, const void *bias,
                              const void *residual, int residual_rows, int64_t residual_ld, void *out, uint32_t *status,
                              cudaStream_t stream, const char **why);

}  // namespace flsm100
