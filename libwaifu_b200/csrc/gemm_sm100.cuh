// Host-side interface of the sm_100a GEMM module: one persistent, warp-specialised tcgen05
// kernel family computing  out[m,n] = epilogue( sum_k A[m,k] * B[n,k] )  with both operands
// K-major ("TN": the activation (m,k) row-major and the weight (n,k) row-major, which is how the
// reference stores a linear layer's weight, flint/cuda/gemm_fp8_cutlass.cu:359-367).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace flsm100 {

enum GemmKind : int {
  kGemmF16 = 0,   // fp16 x fp16 (kind::f16), K a multiple of 8
  kGemmBF16 = 1,  // bf16 x bf16 (kind::f16), K a multiple of 8
  kGemmE4M3 = 2,  // e4m3 x e4m3 (kind::f8f6f4), K a multiple of 16
  kGemmNvf4 = 3,  // e2m1 x e2m1 with unsigned-e4m3 scales per 16 (kind::mxf4nvf4), K a multiple of 32
};

enum Activation : int { kActNone = 0, kActGeluTanh = 1 };

constexpr int kMaxGemmOutputs = 8;

// Status words the kernels write when a bounded wait runs out.
enum : uint32_t {
  kStatusOk = 0,
  kStatusProducerTimeout = 1,
  kStatusMmaTimeout = 2,
  kStatusEpilogueTimeout = 3,
};

struct GemmArgs {
  GemmKind kind;
  int m, n, k;  // k counts elements
  // Operands in device memory, rows 16-byte aligned (pitch = k * element size, a multiple of 16).
  const void *a;  // (m, k)
  const void *b;  // (n, k); with b_is_e4m3 (kGemmF16 only), e4m3 bytes that the kernel widens to half, exactly
  int b_is_e4m3;
  // NVFP4 only: scale factors in the 128-row x 4-factor tile layout the tensor cores read
  // (see pack_scale_factors()), and how many 4-factor tiles one row group holds along k.
  const uint8_t *sfa;
  const uint8_t *sfb;
  int sf_k_tiles;
  // Epilogue, applied in fp32 in this order, then one rounding to the output type:
  //   v = acc * (row_scale[m] * col_scale[n]);  v *= *global_scale;  v += bias[n];
  //   v = act(v);  v += residual[(m % residual_rows) * residual_ld + n]
  const float *row_scale;      // (m) or NULL
  const float *col_scale;      // (n), or (1) when col_scale_scalar, or NULL
  int col_scale_scalar;
  const float *global_scale;   // (1) or NULL
  const void *bias;            // (n) in the output type, or NULL
  const void *residual;        // rows of n in the output type, or NULL
  int residual_rows;           // period of the residual's rows over m (m itself for a full one)
  int64_t residual_ld;
  int act;
  // Row groups (0: none): rows [g * rows_per_group, (g + 1) * rows_per_group) take col_scale and bias
  // from row g of (groups, n) matrices instead of from one (n) vector. rows_per_group is a
  // multiple of 256, so that no tile holds rows of two groups; col_scale is a vector then.
  int rows_per_group;
  // (m) or NULL: the epilogue takes the maximum of |result| over each row, of the values as rounded to
  // the output type, into this array with atomicMax on the float's bits; the caller zeroes it.
  float *row_amax;
  int out_bf16;                // 1 bf16, 0 fp16
  void *out;                   // (m, n), pitch n -- or, with out_ld != 0, columns [out_col0, out_col0 + n)
                               // of a row-major matrix of pitch out_ld
  // Scatter form (the fused all-gather of an output-channel split): up to kMaxGemmOutputs
  // matrices of the same pitch, this GPU's own and its peers' (peer-mapped device memory), each
  // of which receives the tile from the epilogue with plain stores. extra_out[i] may be NULL.
  void *extra_out[7];
  int num_extra_out;
  int64_t out_ld;              // 0: pitch n
  int out_col0;
  uint32_t *status;            // device word, zeroed by the caller; non-zero after a failed wait
  int force_single_cta;        // 1: never pair CTAs (for tests that compare the two forms)
  // Workspace of the stream-K part of the schedule (the K stages of the last, partly filled rounds
  // dealt out evenly over all SMs); without one every tile is computed whole by one unit.
  // sk_partials: room for fp32 accumulator parts, gemm_stream_k_partial_floats() of them at most;
  // sk_counters: words that are zero between launches (the kernel leaves them zero).
  float *sk_partials;
  size_t sk_partial_floats;
  uint32_t *sk_counters;
  size_t sk_counter_words;
  int no_stream_k;             // 1: never use the workspace (for tests that compare the two schedules)
  int no_staged_out;           // 1: results leave by per-lane stores (for measurements that compare the two epilogues)
  cudaStream_t stream;
};

// Launches the GEMM. Returns cudaSuccess or the launch/encode error; `why` then points at a
// static description. Never allocates.
cudaError_t launch_gemm(const GemmArgs &args, const char **why);

// Number of SMs the persistent grid is sized for on the current device.
int sm_count();

// How a product's tiles are dealt out: `dp_rounds` rounds of whole tiles over `units` units
// (tile = round * units + unit), then, from tile `sk_first_tile` on, `sk_tiles` tiles whose
// `num_kb` K stages each are pooled and cut into `units` contiguous runs of equal length (unit u:
// pool positions [total * u / units, total * (u + 1) / units)). sk_tiles is 0 or at least `units`,
// so a run is at least one tile long and a tile is cut into two parts at most.
struct GemmSchedule {
  int units;
  int dp_rounds;
  int sk_tiles;
  int sk_first_tile;
};
GemmSchedule gemm_schedule(int tiles, int max_units, int num_kb, bool allow_stream_k);
// plan[8]: CTAs per unit, BLOCK_N, tiles, K stages per tile, units, dp_rounds, sk_tiles, sk_first_tile
// for a product of the given kind and shape on a device of `sms` SMs. Host arithmetic only.
void gemm_plan(GemmKind kind, int m, int n, int k, int sms, int allow_stream_k, int *plan);

// The most workspace any launch on this device uses for its stream-K part.
size_t gemm_stream_k_partial_floats();
size_t gemm_stream_k_counter_words();

}  // namespace flsm100
