/* flint_sm100.h -- C ABI of libflint_sm100.so: a B200 (sm_100a) implementation of the quantized
 * matmul/linear path of flint, the tensor library of ling0322/libwaifu.
 *
 * Part 1 repeats, signature for signature and value for value, the subset of the reference's
 * flint/capi.h that a caller needs to reach the FP8 product: error reporting, storage, views,
 * transfers and fl_fp8_available / fl_fp8_matmul / fl_fp8_matmul_add. A program (or the Rust FFI
 * in waifu/src/flint/ffi.rs) written against those declarations links against this library
 * unchanged. Each declaration cites the reference interface it replaces as file:line.
 *
 * Part 2 is additive: new enum values appended after the reference's, and new entry points with
 * new names (bf16, per-output-channel scales, dynamic activation quantisation, fused
 * bias/GELU/residual, NVFP4). Nothing in part 1 changes meaning because of it.
 *
 * Conventions (flint/capi.h:20-54): every call returns FL_OK or an error code and leaves a
 * message readable through fl_get_last_error_message() on the calling thread; no exception
 * crosses the boundary. Work on the GPU is enqueued on the legacy default stream and calls
 * return without synchronising (flint/cuda/common.h:51-55); a transfer to the host synchronises.
 */
#ifndef FLINT_SM100_H_
#define FLINT_SM100_H_

#include <stdint.h>

#if defined(_WIN32)
#define FLAPI
#else
#define FLAPI __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ======================= Part 1: the reference's declarations ============================= */

/* flint/capi.h:48-54 */
#define FL_OK 0
#define FL_ERROR_INVALID_ARG 0x0100
#define FL_ERROR_ABORTED 0x0102
#define FL_ERROR_OUT_OF_MEMORY 0x0103

/* flint/capi.h:57-82 */
typedef struct fl_tensor_data_impl_t *fl_tensor_data_t;
typedef struct fl_tensor_view_impl_t *fl_tensor_view_t;
typedef struct fl_operators_impl_t *fl_operators_t;
/* flint/capi.h:71-73. A copy that is still on its way. */
typedef struct fl_transfer_impl_t *fl_transfer_t;

/* flint/capi.h:84-94. 5 and 7 are holes in the reference and stay holes. 11 and 12 are additive. */
typedef enum fl_dtype_t {
  FL_DTYPE_UNKNOWN = 0,
  FL_DTYPE_FLOAT = 1,
  FL_DTYPE_LONG = 2,
  FL_DTYPE_UINT8 = 3,
  FL_DTYPE_FLOAT16 = 4,
  FL_DTYPE_INT8 = 6,
  FL_DTYPE_BOOL = 8,
  FL_DTYPE_INT32 = 9,
  FL_DTYPE_FP8E4M3 = 10,
  /* additive (part 2) */
  FL_DTYPE_BFLOAT16 = 11,
  /* Two e2m1 values per element (one byte): low nibble is the even k. A view's last dimension
   * counts bytes, i.e. k / 2. */
  FL_DTYPE_FP4E2M1X2 = 12,
} fl_dtype_t;

/* flint/capi.h:96-106 */
typedef enum fl_device_type_t {
  FL_DEVICE_CPU = 0,
  FL_DEVICE_CUDA = 1,
  FL_DEVICE_CUDA_HOST = 2,
  FL_DEVICE_METAL = 3,
  FL_DEVICE_VULKAN = 4,
  FL_DEVICE_UNKNOWN = 5,
} fl_device_type_t;

/* flint/capi.h:137-147 */
typedef enum fl_alloc_hint_t {
  FL_ALLOC_ACTIVATION = 0,
  FL_ALLOC_WEIGHT = 1,
  FL_ALLOC_OTHER = 2,
  FL_ALLOC_TEMPORARY_WEIGHT = 3,
} fl_alloc_hint_t;

/* flint/capi.h:151. Picks up the CUDA device; later calls do nothing. */
FLAPI void fl_init(void);
/* flint/capi.h:155. CPU (storage only), CUDA and CUDA_HOST report 1 when a B200-class card exists. */
FLAPI int32_t fl_is_device_available(fl_device_type_t device, int32_t *out);
/* flint/capi.h:158,162 */
FLAPI int32_t fl_get_last_error_code(void);
FLAPI const char *fl_get_last_error_message(void);
/* flint/capi.h:169-175. Only FL_DEVICE_CUDA has operators in this library. */
FLAPI int32_t fl_operators_create(fl_device_type_t device, fl_operators_t *out);
FLAPI void fl_operators_destroy(fl_operators_t operators);
FLAPI int32_t fl_operators_get_device(fl_operators_t operators, fl_device_type_t *out);

/* flint/capi.h:185-213 (storage). On FL_DEVICE_CUDA the memory comes from the device's stream-ordered
 * pool in the compute stream's order and goes back to it the same way, so neither call makes the
 * host or the device wait; only a weight (FL_ALLOC_WEIGHT) of 2 MiB or more gets memory of its own
 * (flint/cuda/cuda_tensor_data.cc:36-77). At most 2^30 elements (flint/tensor.h:41). */
FLAPI int32_t fl_tensor_data_create(fl_device_type_t device, fl_dtype_t dtype, int64_t numel, fl_alloc_hint_t hint,
                                    fl_tensor_data_t *out);
FLAPI int32_t fl_tensor_data_borrow(const void *data, fl_dtype_t dtype, int64_t numel, fl_tensor_data_t *out);
FLAPI void fl_tensor_data_destroy(fl_tensor_data_t data);
FLAPI int32_t fl_tensor_data_get_host_ptr(fl_tensor_data_t data, void **out);

/* flint/capi.h:217-234 (views: shape/stride/offset count elements; stride 0 repeats) */
FLAPI int32_t fl_tensor_view_create(fl_tensor_data_t data, const int32_t *shape, const int32_t *stride, int32_t ndim,
                                    int64_t offset, fl_tensor_view_t *out);
FLAPI void fl_tensor_view_destroy(fl_tensor_view_t view);

/* flint/capi.h:246. src into dest, same shape and dtype, any strides, both on the device. */
FLAPI int32_t fl_copy(fl_operators_t operators, fl_tensor_view_t src, fl_tensor_view_t dest);
/* flint/capi.h:249. Between <float>, <float16> and <bfloat16> here. */
FLAPI int32_t fl_cast(fl_operators_t operators, fl_tensor_view_t input, fl_tensor_view_t out);

/* flint/capi.h:254. Contiguous src -> contiguous dest on another device, same shape and dtype. */
FLAPI int32_t fl_transfer(fl_operators_t operators, fl_tensor_view_t src, fl_tensor_view_t dest);

/* flint/capi.h:256-264. Starts copying contiguous `src`, in page-locked host memory, to `device`
 * (FL_DEVICE_CUDA) and returns before it has arrived. The storage it fills comes back in `dest`,
 * owned by the caller; it must not be read before the transfer has been waited on, and `src`'s
 * storage has to stay alive until then. The copy runs on a stream of its own, beside the kernels. */
FLAPI int32_t fl_transfer_async(fl_tensor_view_t src, fl_device_type_t device, fl_tensor_data_t *dest, fl_transfer_t *out);
/* flint/capi.h:266-268. Orders the work that follows behind the copy, without stopping the caller. */
FLAPI int32_t fl_transfer_wait(fl_transfer_t transfer);
/* flint/capi.h:270-272. The same, but does not return until the copy has finished. */
FLAPI int32_t fl_transfer_wait_sync(fl_transfer_t transfer);
/* flint/capi.h:274-276. Frees the handle, waited on or not. */
FLAPI void fl_transfer_destroy(fl_transfer_t transfer);

/* flint/capi.h:279. <float>, <float16> and <bfloat16> tensors here. */
FLAPI int32_t fl_fill(fl_operators_t operators, fl_tensor_view_t tensor, float value);

/* flint/capi.h:440-446 and 448-456. Matrix multiplication, batched over the leading dimensions:
 * a (..., m, k), b (k, n) or (..., k, n) with leading dimensions that equal a's or are 1, out
 * (..., m, n) contiguous; operands of one type, <float>, <float16> or <bfloat16>, out of that type or
 * <float>; any strides. fl_matmul_add adds `addend`, of out's type, broadcast over out's leading
 * dimensions (a bias (n), or a residual) to the float sum, one rounding (flint/capi.h:448-452).
 * The linear-layer case -- 16-bit a contiguous, b the transposed view (strides 1, k) of a contiguous
 * (n, k) weight (waifu/src/layers.rs:230-246), n and k multiples of 8 -- runs on the tensor cores;
 * every other case on a general fp32-accumulating kernel. */
FLAPI int32_t fl_matmul(fl_operators_t operators, fl_tensor_view_t a, fl_tensor_view_t b, fl_tensor_view_t out);
FLAPI int32_t fl_matmul_add(fl_operators_t operators, fl_tensor_view_t a, fl_tensor_view_t b, fl_tensor_view_t addend,
                            fl_tensor_view_t out);

/* flint/capi.h:480-483. `b` and `out` have `a`'s shape (a broadcast operand is handed over as an
 * expanded view); <float>, <float16> or <bfloat16>, one type; the sum is rounded once. */
FLAPI int32_t fl_add(fl_operators_t operators, fl_tensor_view_t a, fl_tensor_view_t b, fl_tensor_view_t out);

/* flint/capi.h:118-133. Which keys a query may see in fl_attention(): query i sits at position
 * p = i + S - L. */
typedef enum fl_mask_type_t {
  FL_MASK_NONE = 0,           /* every key; block_size 0 */
  FL_MASK_CAUSAL = 1,         /* keys 0..p; block_size 0; needs S >= L */
  FL_MASK_BLOCK_CAUSAL = 2,   /* p's own block of block_size keys and every block before it; needs S >= L */
  FL_MASK_BLOCK_DIAGONAL = 3, /* p's own block alone; needs S == L */
} fl_mask_type_t;

/* flint/capi.h:532-544. Scaled dot product attention: q (N, heads, L, D), k and v (N, kv_heads, S, D)
 * with kv_heads dividing heads, out (N, heads, L, D); <float16> or <bfloat16>, one type. The last
 * dimension is contiguous; the other strides are free (a (N, L, heads, D) tensor transposed is
 * taken as it is) but multiples of 8 elements, and every operand starts on a 16-byte boundary. D is
 * 64 or 128. Softmax in float over scores scaled by 1/sqrt(D); probabilities rounded to the
 * operands' type before the second product (flint/cuda/attention.cu:30-70). A mask that is not one
 * (a block size beside NONE or CAUSAL, none beside a block mask, keys too few) is
 * FL_ERROR_INVALID_ARG, and so is what this library has no kernel for (float32 operands, other
 * head sizes, broadcast q, k or out), with the reason. Blocks of 128 keys no query of a tile sees
 * are skipped. Two
 * launches (a transposition of v into scratch, the attention kernel), no host synchronisation. */
FLAPI int32_t fl_attention(fl_operators_t operators, fl_tensor_view_t q, fl_tensor_view_t k, fl_tensor_view_t v,
                           fl_mask_type_t mask_type, int32_t block_size, fl_tensor_view_t out);

/* flint/capi.h:458-460, flint/capi.cc:1039-1045. 1 for FL_DEVICE_CUDA on compute capability 10.x,
 * 0 for every other device or card, never an error for a missing device. */
FLAPI int32_t fl_fp8_available(fl_device_type_t device, int32_t *out);

/* flint/capi.h:462-468, flint/capi.cc:1047-1053.
 * a <float16>(..., k) times the transpose of data <fp8e4m3>(rows, k) times its one <float> scale,
 * into out <float16>(..., rows). rows a multiple of 8, k of 16. The activation is NOT narrowed:
 * the weight is widened to half and multiplied in half with fp32 accumulation, as the reference
 * does (flint/cuda/gemm_fp8_cutlass.cu:20-29). <bfloat16> a/out is accepted too (additive). */
FLAPI int32_t fl_fp8_matmul(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scale, fl_tensor_view_t out);

/* flint/capi.h:470-478, flint/capi.cc:1055-1097. addend <float16> broadcast over out's leading
 * dimensions: a bias (rows), or a residual; added to the fp32 sum after the scale, one rounding
 * (flint/cuda/gemm_fp8_cutlass.cu:409-426). */
FLAPI int32_t fl_fp8_matmul_add(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scale,
                                fl_tensor_view_t addend, fl_tensor_view_t out);

/* ======================= Part 2: additive entry points ==================================== */

/* Activation applied by the fused epilogue. */
typedef enum fl_activation_t {
  FL_ACT_NONE = 0,
  FL_ACT_GELU_TANH = 1, /* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), waifu/src/krea2/dit.rs:170-188 */
} fl_activation_t;

/* FP8 linear with both operands narrow:
 *   a <float16|bfloat16>(..., k) is quantised on the fly, per row (token): s_m = amax_m / 448,
 *   code = e4m3(a * (1 / s_m)), the reciprocal taken once per row; data <fp8e4m3>(rows, k); scales <float>(rows) per output channel or
 *   <float>(1) per tensor (the reference's format, docs/fp8.md:16-18).
 *   out = round16( act( acc * (s_m * scale_n) + bias_n ) + residual_mn ),   fp32 until the end.
 * bias (rows), residual of out's shape; either may be NULL. rows a multiple of 8, k of 16.
 * No counterpart in the reference, whose activations stay in half. */
FLAPI int32_t fl_fp8_linear(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scales, fl_tensor_view_t bias,
                            fl_tensor_view_t residual, int32_t act, fl_tensor_view_t out);

/* fl_fp8_linear() for callers that must not allocate. It has no counterpart in the reference.
 *
 * Who needs it: a host that runs with every byte of the card already budgeted -- flint's own
 * callers keep weights resident up to a memory limit and evict one when an allocation fails
 * (waifu/src/flint/ir.rs:489-503), so a library that quietly grows a scratch arena behind them can
 * fail or push a weight out -- and a host that cannot afford the device-wide stall a cudaMalloc or
 * cudaFree brings in the middle of a pass. fl_fp8_linear() may grow its arena on any call whose
 * m * k is larger than every earlier one; this entry point never does.
 *
 * How: the quantised activation (m * k bytes), its m row scales and the kernels' status word live
 * in one fixed device array compiled into the library, about 16.3 MiB, which every GPU that loads
 * the library holds until the process ends. The call makes no cudaMalloc, cudaFree, cudaHostAlloc
 * or other allocating call. Arguments and checks are fl_fp8_linear()'s; the arithmetic is the
 * quantiser kernel followed by the product kernel fl_fp8_linear() takes from five rows on (the
 * tcgen05 tile GEMM, or for at most 32 rows against a wide weight the few-row tensor-core kernel)
 * for every row count, so from five rows on the results are bit-identical to fl_fp8_linear()'s, and
 * for one to four rows, where fl_fp8_linear() may take a one-launch few-row kernel with another
 * summation order, they agree within the path's tolerance. FLINT_SM100_SINGLE_CTA and
 * fl_sm100_gemm_timing() do not apply here.
 *
 * Limits, refused with FL_ERROR_INVALID_ARG before anything is launched: at most 65536 activation
 * rows (the product of a's leading dimensions), at most 16 Mi elements in m * k (4352 x 3072 fits),
 * and a weight whose first element is 16-byte aligned (the ordinary entry point would stage it).
 *
 * Sharing: every call on a device uses the same array and finds the last call's bytes in it. The
 * call clears the status word itself and overwrites all codes and scales it reads, so nothing has
 * to be cleared by the caller; but two calls that overlap on the GPU (from two threads, or if this
 * library is ever driven on more than its one stream) race on it and must be serialised by the
 * caller. To report a kernel that gave up on a wait, each call first reads the previous call's
 * status word back, which waits for that call's kernels: consecutive calls do not overlap their
 * launches the way fl_fp8_linear() calls do. The last call's status word is reported by
 * fl_sm100_synchronize() and by a fl_transfer() towards the host.
 *
 * First call: on each device, the first call looks the array's device address up (once, with that
 * device current) and, like any first launch, loads the kernels. Make that first call before
 * beginning any stream capture on that device. (Every call also makes one small synchronous copy
 * on the legacy stream, the read-back above.) */
FLAPI int32_t fl_fp8_linear_static(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scales,
                                   fl_tensor_view_t bias, fl_tensor_view_t residual, int32_t act,
                                   fl_tensor_view_t out);

/* fl_fp8_linear() whose result lands, straight from the GEMM's epilogue, in columns
 * [col0, col0 + rows) of each of `n_dest` (1..8) row-major matrices (..., ld): this GPU's own
 * and, through fl_sm100_ipc_import(), its peers'. This is the all-gather of an output-channel
 * split fused into the product: every rank multiplies by its slice of the weight and writes its
 * column block into every rank's full-width matrix over NVLink with plain stores, tile by tile,
 * while the main loop runs on. The caller orders the ranks afterwards (a barrier or any
 * collective on the stream) before any of them reads the gathered matrix. ld and col0 are
 * multiples of 8. No counterpart in the reference, which runs on one GPU
 * (flint/cuda/cuda_operators.cc:91-96). */
FLAPI int32_t fl_fp8_linear_scatter(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scales,
                                    fl_tensor_view_t bias, fl_tensor_view_t residual, int32_t act,
                                    const fl_tensor_view_t *dests, int32_t n_dest, int32_t col0);

/* The two halves of a narrow gather, for a matrix H = act(a W^T) split over the GPUs by output
 * channel whose next use is another fl_fp8_linear: moving H as e4m3 codes costs half the bytes of
 * moving it in 16 bits, but a row's codes need the row's scale, the maximum over ALL its columns.
 *   fl_fp8_linear_amax: fl_fp8_linear into `out` (this rank's column block, local) that also leaves
 *     in row_amax <float>(rows of a) the largest magnitude of each row of `out` as rounded (the call
 *     clears row_amax first; the epilogue merges with atomicMax).
 *   -- the caller takes the maximum of row_amax over the ranks (one all-reduce of m floats) --
 *   fl_fp8_quantize_scatter: x <float16|bfloat16>(..., k) (the block), quantised per row exactly as
 *     fl_quantize_fp8_activation would quantise the whole row (scale = row_amax / 448), the codes
 *     written into columns [col0, col0 + k) of each of `n_dest` (1..8) <fp8e4m3>(..., ld) matrices:
 *     this GPU's and, through fl_sm100_ipc_import(), its peers', with plain 16-byte stores. Leaves the
 *     rows' scales in row_scales <float>(rows) if that is not NULL. k, ld, col0 multiples of 16.
 * The gathered codes and scales then go to fl_fp8_linear_quantized(), and the result equals the
 * unsplit fl_fp8_linear chain bit for bit. The caller orders the ranks (a barrier or any collective
 * on the stream) between the scatter and the first read. No counterpart in the reference. */
FLAPI int32_t fl_fp8_linear_amax(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scales, fl_tensor_view_t bias,
                                 fl_tensor_view_t residual, int32_t act, fl_tensor_view_t out, fl_tensor_view_t row_amax);
FLAPI int32_t fl_fp8_quantize_scatter(fl_tensor_view_t x, fl_tensor_view_t row_amax, const fl_tensor_view_t *dests,
                                      int32_t n_dest, int32_t col0, fl_tensor_view_t row_scales);
/* The rows' maxima of a block that no GEMM of this library produced (this rank's heads of an
 * attention result, say): row_amax[r] = max |x[r, :]| of x <float16|bfloat16>(rows, k), whose rows
 * may lie further apart than k (a column block of a wider matrix). */
FLAPI int32_t fl_fp8_row_amax(fl_tensor_view_t x, fl_tensor_view_t row_amax);

/* fl_fp8_linear_quantized() with fl_fp8_linear_scatter()'s way out: codes <fp8e4m3>(..., k) and their
 * rows' scales times the weight, the product written into columns [col0, col0 + rows) of each of
 * `n_dest` (1..8) <float16|bfloat16>(..., ld) matrices, whose type is the product's. The second GEMM
 * of a column-split MLP whose hidden activation was gathered as codes. */
FLAPI int32_t fl_fp8_linear_quantized_scatter(fl_tensor_view_t codes, fl_tensor_view_t row_scales, fl_tensor_view_t data,
                                              fl_tensor_view_t scales, fl_tensor_view_t bias, fl_tensor_view_t residual,
                                              int32_t act, const fl_tensor_view_t *dests, int32_t n_dest, int32_t col0);

/* A barrier among the GPUs of one box (one process each), in one small kernel on the stream, that can
 * carry a maximum per row: what stands between the kernels of a split linear in place of a library
 * collective. mailboxes[i] is rank i's <int32>(n_ranks, FL_SM100_PEER_HEADER + capacity) matrix, zeroed
 * when made: mailboxes[rank] this GPU's own (FL_ALLOC_WEIGHT storage of 2 MiB or more, exported), the
 * others imported with fl_sm100_ipc_import(). Every rank makes the same calls in the same order with
 * the same `epoch`, 1 at the first call and larger at every later one. The kernel
 *   - if row_amax <float>(rows <= capacity) is not NULL, writes it into every rank's mailbox;
 *   - makes everything this GPU wrote before it (earlier kernels of the stream included: scattered
 *     codes, a product's column block) visible ahead of its flag, and sets the flag in every mailbox;
 *   - waits until every rank's flag in its own mailbox has reached `epoch`: what those ranks wrote
 *     before their call is visible to the kernels that follow on this stream;
 *   - if row_amax, leaves in it the largest of the ranks' values per row.
 * The wait is bounded: after max_polls polls (0: a default of about two seconds) the kernel records
 * a status the next call and fl_sm100_synchronize() report as FL_ERROR_ABORTED, and returns with
 * row_amax as it was. A rank may not reuse what a peer reads (the scattered buffers) before a later
 * exchange has completed. No counterpart in the reference. */
#define FL_SM100_PEER_HEADER 64
FLAPI int32_t fl_sm100_peer_exchange(const fl_tensor_view_t *mailboxes, int32_t n_ranks, int32_t rank, int32_t epoch,
                                     fl_tensor_view_t row_amax, int32_t max_polls);

/* Device storage shared between the processes of one box (one process per GPU): export writes
 * the 64-byte handle of storage made by fl_tensor_data_create(FL_DEVICE_CUDA, ..., FL_ALLOC_WEIGHT, ...)
 * of 2 MiB or more (memory of its own; blocks of the stream-ordered pool have no handle); import maps
 * another process's storage here (peer access over NVLink); fl_tensor_data_destroy() unmaps. */
FLAPI int32_t fl_sm100_ipc_export(fl_tensor_data_t data, void *handle_out);
FLAPI int32_t fl_sm100_ipc_import(const void *handle, fl_dtype_t dtype, int64_t numel, fl_tensor_data_t *out);

/* 1 where fl_nvfp4_linear can run (the same cards as fl_fp8_available). */
FLAPI int32_t fl_nvfp4_available(fl_device_type_t device, int32_t *out);

/* NVFP4 linear:
 *   codes <fp4e2m1x2>(rows, k/2); block_scales <fp8e4m3>(rows, k/16), unsigned, one per 16
 *   consecutive k; global_scale <float>(1). a is quantised on the fly per 16-element block:
 *   s = e4m3(amax_block / 6), code = e2m1(a * (1 / s)), global 1.
 *   out = round16( act( acc * global_scale + bias_n ) + residual_mn ).
 * rows a multiple of 8, k of 32. No counterpart in the reference (it has no FP4 of any kind). */
FLAPI int32_t fl_nvfp4_linear(fl_tensor_view_t a, fl_tensor_view_t codes, fl_tensor_view_t block_scales,
                              fl_tensor_view_t global_scale, fl_tensor_view_t bias, fl_tensor_view_t residual,
                              int32_t act, fl_tensor_view_t out);

/* Device-side weight preparation, the rule of tools/model_writer.py:143-174 applied per row:
 * w <float>(rows, k) -> codes <fp8e4m3>(rows, k), scales <float>(rows). */
FLAPI int32_t fl_quantize_fp8_rows(fl_tensor_view_t w, fl_tensor_view_t codes, fl_tensor_view_t scales);
/* w <float>(rows, k) -> NVFP4 codes, block scales and the global scale (amax / (448 * 6)). */
FLAPI int32_t fl_quantize_nvfp4(fl_tensor_view_t w, fl_tensor_view_t codes, fl_tensor_view_t block_scales,
                                fl_tensor_view_t global_scale);
/* The dynamic activation quantiser on its own (what fl_fp8_linear applies to `a`), for tests:
 * a <float16|bfloat16>(m, k) -> codes <fp8e4m3>(m, k), scales <float>(m). */
FLAPI int32_t fl_quantize_fp8_activation(fl_tensor_view_t a, fl_tensor_view_t codes, fl_tensor_view_t scales);

/* The step before a block's projection, fused with its quantiser (the consumer the reference
 * builds from layer_norm, mul, add and cast nodes: waifu/src/qwen_image/dit.rs:179-184, over
 * flint's layerNorm, flint/cpu/normalizations.cc:98-140): per row of x <float16|bfloat16>(..., k),
 *   n = (x - mean) * (1 / sqrt(var + eps))    fp32 sums; mean = sum / k, var = sumsq / k - mean^2
 *                                             (eps alone where that is not positive), no affine
 *   h = round16( n * scale_g + n + shift_g )  scale, shift: (k) or (groups, k) of x's type (the rows
 *                                             contiguous, any stride between them), or NULL;
 *                                             row r belongs to group r / (rows / groups)
 *   codes, row_scales = per-row e4m3 of h     exactly fl_quantize_fp8_activation(h)
 * One pass over x; h is never written. codes <fp8e4m3> of x's shape, row_scales <float>(rows). */
FLAPI int32_t fl_fp8_layernorm_quantize(fl_tensor_view_t x, fl_tensor_view_t scale, fl_tensor_view_t shift, float eps,
                                        fl_tensor_view_t codes, fl_tensor_view_t row_scales);
/* The step between a gated MLP's two projections, fused with the second one's quantiser: flint's
 * swiglu (flint/cpu/glu.cc:36-67; the first half of the last dimension is the gate, the second the
 * value) on x <float16|bfloat16>(..., 2 h),
 *   y = round16( g / (1 + exp(-g)) * v )
 * then codes, row_scales = per-row e4m3 of y (..., h), exactly fl_quantize_fp8_activation(y).
 * One pass over x; y is never written. */
FLAPI int32_t fl_fp8_swiglu_quantize(fl_tensor_view_t x, fl_tensor_view_t codes, fl_tensor_view_t row_scales);
/* fl_fp8_linear for an activation that is quantised already (by fl_fp8_layernorm_quantize or
 * fl_quantize_fp8_activation): codes <fp8e4m3>(..., k) with row_scales <float>(rows); out
 * <float16|bfloat16>(..., n) chooses the type of bias, residual and result. */
FLAPI int32_t fl_fp8_linear_quantized(fl_tensor_view_t codes, fl_tensor_view_t row_scales, fl_tensor_view_t data,
                                      fl_tensor_view_t scales, fl_tensor_view_t bias, fl_tensor_view_t residual,
                                      int32_t act, fl_tensor_view_t out);

/* fl_fp8_linear_quantized with row groups: rows [g * rows_per_group, (g + 1) * rows_per_group) of the
 * left operand take their per-channel scales and bias from row g of `scales` <float>(groups, rows)
 * and `bias` (groups, rows) -- a gate per image folded into the scales and the bias of one product
 * (x + gate * linear(a): waifu/src/qwen_image/dit.rs:322-335) without one launch per image.
 * rows_per_group is a multiple of 256 (no tile of the product holds rows of two groups). */
FLAPI int32_t fl_fp8_linear_quantized_grouped(fl_tensor_view_t codes, fl_tensor_view_t row_scales, fl_tensor_view_t data,
                                              fl_tensor_view_t scales, fl_tensor_view_t bias, fl_tensor_view_t residual,
                                              int32_t act, int32_t rows_per_group, fl_tensor_view_t out);

/* The step between the fused q/k/v projection and attention, in place on the projection's output
 * qkv <float16|bfloat16>(..., 3 * heads * head_dim) (q heads, k heads, v heads along the last
 * dimension; head_dim 64, 128 or 256; every operand 16-byte aligned): per row and q or k head,
 *   n = round16( x * w * (1 / sqrt(mean(x^2) + eps)) )   flint's rmsNorm, flint/cpu/normalizations.cc:33-70,
 *                                                   one reciprocal per head instead of a division per
 *                                                   element; w = q_weight / k_weight (head_dim) or NULL
 *   (n_2j, n_2j+1) <- round16( n_2j cos_j - n_2j+1 sin_j,  n_2j sin_j + n_2j+1 cos_j )
 *                                                   waifu/src/krea2/dit.rs:260-275
 * with cos, sin <float>(tokens, head_dim / 2) and row r at position r % tokens. v is left as it
 * is, so attention can read q, k and v as strided views of the one buffer. */
FLAPI int32_t fl_qk_norm_rope(fl_tensor_view_t qkv, fl_tensor_view_t q_weight, fl_tensor_view_t k_weight,
                              fl_tensor_view_t cos, fl_tensor_view_t sin, float eps, int32_t heads);

/* The plan the few-row kernel (at most 16 activation rows) would run a shape with; host arithmetic
 * only, no GPU needed, so that its index arithmetic can be checked anywhere. weight_bytes 1 (e4m3)
 * or 2 (16-bit), activation_bytes 1 (quantised rows) or 2. plan[16]: [0] CTAs per SM (0: the shape
 * goes to the tile kernel and the rest is 0), [1] channels per unit, [2] K slices per stage,
 * [3] stages per unit, [4] weight bytes of a stage per channel, [5] of a slice, [6] K positions a
 * step can touch (in weight bytes), [7] bytes between channels in a stage, [8] bytes of a stage,
 * [9] ring depth, [10] one bulk copy per stage, [11] bytes between activation rows, [12] bytes of
 * the activation rows, [13] of the staged epilogue operands, [14] CTAs, [15] dynamic shared
 * memory of a CTA. */
FLAPI int32_t fl_sm100_few_rows_plan(int32_t m, int32_t n, int32_t k, int32_t weight_bytes, int32_t activation_bytes,
                                     int32_t has_residual, int32_t *plan);

/* Which kernel a product of few rows takes by its shape alone (operands aligned, the environment's
 * switches unset); host arithmetic only, no GPU needed. entry 0: fl_fp8_matmul[_add] with half
 * rows, 1: fl_fp8_linear (and _static, _quantized), 2: fl_matmul[_add] on 16-bit operands; n the
 * weight's rows (output channels). Returns 2: a tensor-core few-row kernel (the weight on the M side
 * of the instruction), 1: the mma.sync few-row kernel, 0: the tile kernel; -1 for a bad argument. */
FLAPI int32_t fl_sm100_few_rows_route(int32_t entry, int32_t m, int32_t n, int32_t k);

/* Which tile kernel a product of `kind` (0 half, 1 bfloat16, 2 e4m3, 3 nvfp4) and shape would run on
 * and how its tiles are dealt out over a device of `sms` SMs; host arithmetic only, no GPU needed, so
 * that the schedule can be checked anywhere. plan[8]: [0] CTAs per unit (2: a cluster pair sharing a
 * 256-row tile), [1] tile width, [2] tiles, [3] K stages (128 bytes of K each) per tile, [4] units,
 * [5] rounds of whole tiles (tile = round * units + unit), [6] tiles of the stream-K part that
 * follows, from tile [7] on: their K stages are pooled and unit u computes pool positions
 * [total * u / units, total * (u + 1) / units), total = [6] * [3]. [6] is 0 (no such part: the last
 * round is simply partly filled) or at least [4]. */
FLAPI int32_t fl_sm100_gemm_plan(int32_t kind, int32_t m, int32_t n, int32_t k, int32_t sms, int32_t allow_stream_k,
                                 int32_t *plan);

/* Storage over device memory the caller already owns (for instance a torch tensor's): nothing
 * is copied and nothing is freed on destroy. The device counterpart of fl_tensor_data_borrow(). */
FLAPI int32_t fl_tensor_data_borrow_device(void *device_ptr, fl_dtype_t dtype, int64_t numel, fl_tensor_data_t *out);

/* The download fl_transfer_async() has no counterpart for in the reference (whose device-to-host copy
 * is synchronous, flint/cuda/to_device.cc:60-66): contiguous device `src` into page-locked host
 * `dest` of the same shape and dtype, on a stream of its own, ordered behind the work queued so far.
 * The host may read `dest` once fl_transfer_wait_sync() on the handle has returned; `src` has to
 * stay alive until then. Free the handle with fl_transfer_destroy(). */
FLAPI int32_t fl_sm100_transfer_to_host_async(fl_tensor_view_t src, fl_tensor_view_t dest, fl_transfer_t *out);

/* Selects the CUDA device of this process (one process per GPU). Allowed before the first
 * operation, or again with the same ordinal; a second device in one process is refused. */
FLAPI int32_t fl_sm100_set_device(int32_t ordinal);
/* Waits for the default stream, then reports the kernels' status word (the library's, and the one
 * fl_fp8_linear_static()'s kernels use): 0, or the code of the bounded wait that gave up inside a
 * kernel (the call then also returns FL_ERROR_ABORTED). */
FLAPI int32_t fl_sm100_synchronize(int32_t *kernel_status);
/* Per-launch timing of the GEMM kernel alone: while enabled, every GEMM launch is bracketed by
 * CUDA events on its stream; fl_sm100_gemm_timing_read() waits for the stream, returns the summed
 * kernel time and the number of launches since the last read, and clears them. For benchmarks. */
FLAPI int32_t fl_sm100_gemm_timing(int32_t enable);
FLAPI int32_t fl_sm100_gemm_timing_read(double *total_ms, int64_t *launches);
/* How many kernels of this library the calling process has launched so far. */
FLAPI int64_t fl_sm100_launch_count(void);

/* Self-tests of the error path, for this library's own tests. Neither faults nor hangs anything.
 * fl_sm100_selftest_wait_timeout() launches one warp that waits, with a limit of `polls` (1..4096)
 * polls, on a barrier nothing ever arrives on, and reports status 0x51 the way the GEMM and attention
 * kernels report a wait that gave up: the next fl_sm100_synchronize() returns FL_ERROR_ABORTED with
 * that status, and the call after it succeeds. fl_sm100_selftest_set_static_status() writes `code`
 * into the status word of fl_fp8_linear_static()'s array, as one of its kernels would. */
FLAPI int32_t fl_sm100_selftest_wait_timeout(int32_t polls);
FLAPI int32_t fl_sm100_selftest_set_static_status(uint32_t code);

#ifdef __cplusplus
}
#endif

#endif /* FLINT_SM100_H_ */
