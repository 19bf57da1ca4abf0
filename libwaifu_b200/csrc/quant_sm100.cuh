// Bandwidth-shaped helper kernels around the GEMM: the dynamic activation quantisers, the
// device-side weight quantisers, the scale-factor re-tiling NVFP4 needs, and the e4m3 -> half
// widening of the reference-compatible path. None of them allocates.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

// Per-row (token) e4m3: scales[r] = amax_r / 448, codes = e4m3_rn_sat(x * (1 / scales[r])) with
// one IEEE reciprocal per row; a zero row gives scale 0 and codes 0 (the zero rule of
// tools/model_writer.py:162-170). The weight quantiser below divides, as that recipe does.
cudaError_t quantize_fp8_act(const void *x, int is_bf16, int m, int k, uint8_t *codes, float *scales,
                             cudaStream_t stream);
cudaError_t quantize_fp8_rows_f32(const float *w, int rows, int k, uint8_t *codes, float *scales,
                                  cudaStream_t stream);

// quantize_fp8_act with the rows' maxima given instead of taken (`amax` (m): the maximum of |x| over
// a row that may be wider than x), the codes written into columns [col0, col0 + k) of `n_dest`
// (1..8) matrices of pitch `ld` bytes, and scales[r] = amax[r] / 448 (scales may be null). k, ld and
// col0 multiples of 16, every base 16-byte aligned.
cudaError_t quantize_fp8_scatter(const void *x, int is_bf16, int m, int k, const float *amax, uint8_t *const *dests,
                                 int n_dest, int64_t ld, int col0, float *scales, cudaStream_t stream);

// amax[r] = the largest |x[r, :]| of an (m, k) 16-bit matrix whose rows lie `pitch` elements apart
// (NaNs order above every number, as in the epilogue's row maxima).
cudaError_t row_amax_16(const void *x, int is_bf16, int m, int k, int64_t pitch, float *amax, cudaStream_t stream);

// Layer norm over the last dimension (no affine; fp32 sums, mean = sum / k, variance =
// sumsq / k - mean^2, eps inside the root: flint/cpu/normalizations.cc:98-140), then the adaLN modulation
// h = round16(n * scale + n [+ shift]) with `scale`/`shift` (groups, k) 16-bit or null, a group's
// row `scale_pitch` / `shift_pitch` elements after the previous one's, and row r in group
// r / rows_per_group (waifu/src/qwen_image/dit.rs:179-184), then per-row e4m3 of h
// exactly as quantize_fp8_act. One pass over x; the modulated row never reaches memory.
cudaError_t ln_modulate_quantize_fp8(const void *x, int is_bf16, int m, int k, const void *scale, int64_t scale_pitch,
                                     const void *shift, int64_t shift_pitch, int rows_per_group, float eps,
                                     uint8_t *codes, float *row_scales, cudaStream_t stream);

// Scale factors of a (rows, k/16) operand in the tile layout the block-scaled MMA reads: tiles
// of 128 rows x 4 factors (512 bytes), byte (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4) of
// tile (r / 128, b / 4); tiles of one row group are consecutive, `sf_k_tiles` per group.
inline int sf_k_tiles_for(int k) { return ((k / 16 + 3) / 4 + 3) / 4 * 4; }
inline int64_t sf_tiled_bytes(int rows, int k, int extra_groups) {
  return static_cast<int64_t>((rows + 127) / 128 + extra_groups) * sf_k_tiles_for(k) * 512;
}

// Per-16-block e2m1 with unsigned-e4m3 block scales, global scale 1; codes (m, k/2) row-major,
// scale factors written straight into the tile layout (`sf_tiled` zeroed by the caller).
cudaError_t quantize_nvfp4_act(const void *x, int is_bf16, int m, int k, uint8_t *codes, uint8_t *sf_tiled,
                               cudaStream_t stream);
// What fl_nvfp4_linear needs ahead of its GEMM, in one launch: the activation's codes and tiled
// scale factors (quantize_nvfp4_act) and the weight's plain (rows, k/16) block scales in the tile
// layout with `w_extra_groups` spare row groups (pack_scale_factors), padding written as zeros, so
// neither destination has to be cleared first.
cudaError_t nvfp4_prepare(const void *x, int is_bf16, int m, int k, uint8_t *codes, uint8_t *sfa_tiled,
                          const uint8_t *wsf_plain, int rows, int w_extra_groups, uint8_t *sfb_tiled, cudaStream_t stream);
// NVFP4 weight from fp32: global = amax / (448 * 6); plain (rows, k/16) block scales.
// `amax_word` is a device word used for the reduction.
cudaError_t quantize_nvfp4_weight_f32(const float *w, int rows, int k, uint8_t *codes, uint8_t *sf_plain,
                                      float *global_scale, uint32_t *amax_word, cudaStream_t stream);
// Plain (rows, k/16) scale factors -> tile layout (`sf_tiled` zeroed by the caller).
cudaError_t pack_scale_factors(const uint8_t *sf_plain, int rows, int k, uint8_t *sf_tiled, cudaStream_t stream);

// flint's swiglu (first half of the last dimension the gate, second the value; silu(g) * v in fp32,
// narrowed to 16 bits: flint/cpu/glu.cc:36-67) on x (m, 2 h), then per-row e4m3 of the (m, h)
// result exactly as quantize_fp8_act. One pass; the gated row never reaches memory.
cudaError_t swiglu_quantize_fp8(const void *x, int is_bf16, int m, int h, uint8_t *codes, float *row_scales,
                                cudaStream_t stream);

// codes -> fp16 / bf16 values (exact), the widening flint's kernel does in registers
// (flint/cuda/gemm_fp8_cutlass.cu:20-29).
cudaError_t widen_e4m3(const uint8_t *codes, int64_t numel, void *out16, int out_bf16, cudaStream_t stream);

// Strided gather of a 16-bit view into a contiguous buffer (for addends no epilogue can index).
cudaError_t expand_16(const void *src, const int32_t *shape, const int64_t *stride, int ndim, void *dst,
                      cudaStream_t stream);

int64_t helper_launch_count();

}  // namespace flsm100
