/* TEST INFRASTRUCTURE -- not product code.
 *
 * A plain-C, CPU-only restatement of the arithmetic of flint's quantized linear, used only as
 * the checker of the CUDA path (tests, the smoke check and the CPU-baseline leg of the bench).
 * Nothing in the product library links, loads or calls this file.
 *
 * Pinning: the e4m3 decode, the per-tensor quantizer, the "scale then addend, one rounding"
 * epilogue and the known-answer vectors of the reference's own tests are checked against this
 * file by the CPU test-suite. The bf16, per-channel, per-token, GELU and NVFP4 parts have no
 * counterpart in the reference's tests: for them parity is pinned only against torch /
 * ml_dtypes casts and the reference's float32 CPU GEMM ("parity unpinned" by the reference).
 *
 * Citations are paths inside the reference project (ling0322/libwaifu).
 */
#ifndef FLINT_ORACLE_H_
#define FLINT_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar codecs -------------------------------------------------------------------- */

/* OCP e4m3fn code -> value. Follows flint/cuda/gemm_fp8_cutlass_test.cc:95-102 (bias 7,
 * subnormals m*2^-9, no infinities); 0x7f/0xff decode to NaN as flint/dtype.h:80-86 says. */
float fo_e4m3_decode(uint8_t code);
/* value -> e4m3fn code, round-to-nearest-even, saturating to +-448, NaN -> 0x7f. The rounding
 * of tools/model_writer.py:170-172 (clamp, then torch's float8_e4m3fn cast). */
uint8_t fo_e4m3_encode(float x);
/* e2m1 nibble (bit3 sign; magnitudes 0,0.5,1,1.5,2,3,4,6) <-> value, RNE saturating to +-6. */
float fo_e2m1_decode(uint8_t nibble);
uint8_t fo_e2m1_encode(float x);
/* bfloat16 / float16 round-to-nearest-even. bf16 follows waifu/src/qwen_image/pipeline.rs:69-76. */
uint16_t fo_bf16_from_f32(float x);
float fo_bf16_to_f32(uint16_t h);
uint16_t fo_f16_from_f32(float x);
float fo_f16_to_f32(uint16_t h);

/* ---- quantizers ------------------------------------------------------------------------ */

/* tools/model_writer.py:143-174: scale = amax/448 (fp32), zero tensor -> divisor 1, scale 0. */
void fo_quantize_fp8_tensor(const float *w, int64_t numel, uint8_t *codes, float *scale);
/* The same rule applied to each row on its own (one fp32 scale per output channel). */
void fo_quantize_fp8_rows(const float *w, int rows, int k, uint8_t *codes, float *scales);
/* Dynamic per-token quantisation of a 16-bit activation (is_bf16: 1 bf16, 0 fp16):
 * amax over the row in fp32, scale = amax/448, code = e4m3(x * (1/scale)) with the reciprocal
 * taken once per row in IEEE fp32; zero row -> scale 0, codes 0. */
void fo_quantize_fp8_act(const uint16_t *x, int is_bf16, int rows, int k, uint8_t *codes,
                         float *scales);
/* The same with the rows' maxima given: one rank's column block of a row whose maximum was taken
 * over all ranks' blocks. codes (rows, k), scales[r] = amax[r] / 448. */
void fo_quantize_fp8_act_amax(const uint16_t *x, int is_bf16, int rows, int k, const float *amax,
                              uint8_t *codes, float *scales);
/* NVFP4 weight: g = amax/(448*6); per 16 consecutive k: s = e4m3(amax_b/(6 g)) (unsigned),
 * code = e2m1(w * (1/(decode(s) g))), the reciprocal taken once per block in IEEE fp32; zero
 * block -> s = 0, codes 0. codes: two per byte, low nibble
 * is the even k. block_scales (rows, k/16) row-major. k must be a multiple of 16. */
void fo_quantize_nvfp4_weight(const float *w, int rows, int k, uint8_t *codes,
                              uint8_t *block_scales, float *global_scale);
/* NVFP4 activation from 16-bit input, global scale 1: s = e4m3(amax_b/6), code = e2m1(x * (1/s)). */
void fo_quantize_nvfp4_act(const uint16_t *x, int is_bf16, int rows, int k, uint8_t *codes,
                           uint8_t *block_scales);

/* ---- decoders to float32 (exact) ------------------------------------------------------ */
void fo_decode_e4m3(const uint8_t *codes, int64_t numel, float *out);
/* out[r,k] = e2m1(code) * e4m3(block scale) -- exact in fp32 (at most 2+4 mantissa bits). */
void fo_decode_nvfp4(const uint8_t *codes, const uint8_t *block_scales, int rows, int k,
                     float *out);
void fo_widen_16(const uint16_t *x, int is_bf16, int64_t numel, float *out);
/* float32 -> bf16 / fp16 bit patterns, round to nearest even (the scalar helpers above, over an array). */
void fo_narrow_16(const float *x, int is_bf16, int64_t numel, uint16_t *out);

/* ---- the products ---------------------------------------------------------------------- */

/* C[m,n] = sum_k A[m,k] * B[n,k], fp32 accumulate in k order within 8 interleaved partial sums.
 * The stand-in for the reference's fl_matmul (flint/cpu/matmul.cc:306-322) where the reference
 * build is not available. OpenMP over rows of C. */
void fo_gemm_f32_nt(const float *a, const float *b, float *c, int m, int n, int k);
/* The same in double, for a stricter check on small cases
 * (flint/metal_native/operators_test.cc:1391-1398). */
void fo_gemm_f64_nt(const float *a, const float *b, double *c, int m, int n, int k);

#define FO_ACT_NONE 0
#define FO_ACT_GELU_TANH 1

/* The epilogue, element by element, in fp32 with one rounding at the end:
 *   v = acc[m,n] * row_scale[m] * col_scale[n]   (row_scale NULL -> 1; col_scale_count 1 -> one
 *                                                 scale for the tensor)
 *   v = v * global_scale                          (NVFP4 only; pass 1.0f otherwise)
 *   v += bias[n]                                  (NULL -> none)
 *   v = gelu_tanh(v)                              (act == FO_ACT_GELU_TANH;
 *                                                  waifu/src/krea2/dit.rs:170-188)
 *   v += residual[m,n]                            (NULL -> none)
 *   out = rn_16(v)
 * Order "scale, then addend, one rounding": flint/cuda/gemm_fp8_cutlass.cu:107-125,154-168. */
void fo_epilogue(const float *acc, int m, int n, const float *row_scale, const float *col_scale,
                 int col_scale_count, float global_scale, const uint16_t *bias,
                 const uint16_t *residual, int act, int out_is_bf16, uint16_t *out);

#ifdef __cplusplus
}
#endif

#endif /* FLINT_ORACLE_H_ */
