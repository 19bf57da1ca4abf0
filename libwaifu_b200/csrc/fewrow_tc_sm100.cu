// At most 16 activation rows against an e4m3 weight that is widened exactly to half (flint's
// fl_fp8_matmul, flint/cuda/gemm_fp8_cutlass.cu): a product bound by streaming the weight from HBM
// once. Here the weight sits on the M side of tcgen05.mma and the rows are its N = 16, so that no
// instruction of a CUDA core multiplies anything and the time does not depend on the row count
// (the kernel in skinny_sm100.cu, which multiplies on mma.sync, takes 20 us for one row against
// 16384 x 3072 and 36 us for sixteen; this one 12.0 to 12.5 us). The widened weight never
// touches shared memory: the A operand of tcgen05.mma may lie in tensor memory (row i of the tile
// in lane i, the sixteen halves of an instruction packed into eight columns), so shared memory
// holds nothing but bytes as they came from HBM, six stages of 32 KB in flight per CTA.
//   warp 8     producer: per stage of 256 K positions two TMA copies of 128 weight rows x 128 e4m3
//              bytes (128-byte swizzle) into a ring of six raw stages, and four copies of the 16 rows
//              x 128 bytes of x (128-byte swizzle) into a ring of four; the weight is read exactly once;
//   warps 0-7  converters: a thread owns one of the 128 channels (warp % 4 is the quarter of tensor
//              memory's lanes the warp may write, warp / 4 the half of the stage), reads 128 e4m3
//              bytes of its row from the raw tile (the swizzle puts the 32 rows a warp reads in one
//              instruction into different banks), widens them in registers (cvt.rn.f16x2.e4m3x2,
//              exact), writes them with tcgen05.st into one of three units of 128 columns, and hands
//              the raw stage back;
//   warps 9-12 four threads issue the sixteen tcgen05.mma kind::f16 (M = 128 channels, N = 16 rows,
//              K = 16) of a stage, four each, into an accumulator each. Every tcgen05
//              issue costs the issuing thread some 60 cycles: with one thread issuing all sixteen
//              the kernel took 16.9 us, with two 14.0 us, with four 12.7 us;
//   warps 0-3  then the epilogue: a lane owns a channel, reads its 4 x 16 partial sums and adds them;
//              scale, bias, residual, one rounding; for every row the warp stores 32 consecutive
//              channels.
// A CTA owns 128 output channels and is paced by its own chain (load, widen, multiply) over the
// k / 256 stages, some 0.65 us each after 4.5 us of launch, first load and epilogue: 11 to 12.5 us at
// k = 3072 for any channel count up to 148 x 128. Sixteen converter warps, on alternate stages or
// on quarters of every stage, were no faster. Every wait is bounded (status word, as everywhere else).
#include "fewrow_tc_sm100.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

constexpr int kChannels = 128;   // per CTA: the M of the instruction
constexpr int kTokens = 16;      // its N, or twice that (the template parameter of the kernels below)
constexpr int kBlockK = 64;      // K positions per block: 128 bytes of an x row, four instructions
constexpr int kBlocksPerStage = 4;
constexpr int kStageK = kBlocksPerStage * kBlockK;     // K positions per ring stage
constexpr int kRawWBytes = kChannels * kStageK;        // 32 KB
constexpr int kAtomBytes = kChannels * 128;            // 128 rows x 128 e4m3 bytes, 128-byte swizzle
constexpr int kAtoms = kStageK / 128;                  // 2 per stage
constexpr int kUnitCols = kStageK / 2;                 // 128 columns: 256 halves of a row, two to a column
constexpr int kMmaWarps = 4;                           // W: threads that issue, one block of a stage each
constexpr int kChains = 1;                             // C: accumulators per issuing thread (two in turn measured the same)
constexpr int kTmemCols = 512;                         // 64 or 128 + 3 x 128; allocations are powers of two
constexpr int kConvGroups = kAtoms;                    // warps 0..7 in groups of four
constexpr int kConvWarps = 4 * kConvGroups;
constexpr int kProducer = kConvWarps;
constexpr int kMma = kProducer + 1;
constexpr int kThreads = (kMma + kMmaWarps) * 32;
constexpr int kRawOff = 0;
static_assert(kBlocksPerStage % kMmaWarps == 0, "the blocks of a stage are dealt evenly");

// What depends on the rows an instruction takes (NTOK = 16, 32 or 64): the instruction's time does
// not, so 32 rows cost what one costs. Shared memory (227 KB) and tensor memory (512 columns) are
// dealt accordingly.
template <int NTOK>
struct TcCfg {
  static constexpr int kXAtomBytes = NTOK * kBlockK * 2;             // 2, 4 or 8 KB: a block's rows x 128 bytes
  static constexpr int kXBytes = kBlocksPerStage * kXAtomBytes;      // 8, 16 or 32 KB
  // Raw weight stages are given back as soon as they are widened, stages of x only when the
  // instructions that read them are done: x needs its four (with two of 64 rows, 64 x 16384 x 3072
  // took 18.6 us, with three 15.9, with four 15.0), the weight gets what is left.
  static constexpr int kRawStages = NTOK == 16 ? 6 : NTOK == 32 ? 5 : 3;
  static constexpr int kXStages = 4;
  static constexpr int kUnits = NTOK == 64 ? 2 : 3;                  // widened stages in tensor memory (two measured the same as three)
  static constexpr int kAccCols = kMmaWarps * kChains * NTOK;        // 64, 128 or 256 columns
  static constexpr int kUnitCol0 = kAccCols;
  static constexpr int kXOff = kRawOff + kRawStages * kRawWBytes;
  static constexpr int kSmemBytes = kXOff + kXStages * kXBytes + 1024;
  static_assert(kUnitCol0 + kUnits * kUnitCols <= kTmemCols, "tensor memory");
  static_assert(kXBytes % 1024 == 0 && kAtomBytes % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
  static_assert(kSmemBytes <= 227 * 1024 - 512, "shared memory");
};

struct Params {
  const float *scale;
  const void *bias;
  const void *residual;
  int residual_rows;
  long long residual_ld;
  void *out;
  int m, n, k;
  int cpc;  // channels per CTA: at most 128, a multiple of 8
  uint32_t *status;
};

template <int NTOK>
__global__ void __launch_bounds__(kThreads, 1)
fewrow_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const Params p) {
  using C = TcCfg<NTOK>;
  constexpr int kRawStages = C::kRawStages, kXBytes = C::kXBytes, kXAtomBytes = C::kXAtomBytes, kXOff = C::kXOff;
  constexpr int kUnitCol0 = C::kUnitCol0, kXStages = C::kXStages, kUnits = C::kUnits;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t raw_full_bar[kRawStages], raw_empty_bar[kRawStages];
  __shared__ __align__(8) uint64_t x_full_bar[kXStages], x_empty_bar[kXStages];
  __shared__ __align__(8) uint64_t unit_full_bar[kUnits], unit_empty_bar[kUnits];
  __shared__ __align__(8) uint64_t acc_full_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile uint32_t abort_flag;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * p.cpc;
  const int num_kb = p.k / kBlockK;
  const int num_stages = (num_kb + kBlocksPerStage - 1) / kBlocksPerStage;

  if (warp == 0) {  // (a lane per ring slot: 27 barriers set up one after the other were half a microsecond)
    if (lane < kRawStages) {
      mbar_init(&raw_full_bar[lane], 1);
      mbar_init(&raw_empty_bar[lane], kConvWarps);
    }
    if (lane < kXStages) {
      mbar_init(&x_full_bar[lane], 1);
      mbar_init(&x_empty_bar[lane], kMmaWarps);
    }
    if (lane < kUnits) {
      mbar_init(&unit_full_bar[lane], kConvWarps);
      mbar_init(&unit_empty_bar[lane], kMmaWarps);
    }
    if (lane == 0) {
      abort_flag = 0;
      mbar_init(&acc_full_bar, kMmaWarps);
    }
    fence_barrier_init();
  }
  if (warp == kProducer && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    // The first stages of the weight are asked into L2 before the kernel ahead in the stream is
    // known to be done: a prefetch writes nothing, and if that kernel does write these bytes its
    // stores land in the same L2, so the loads below read what they would have read anyway. The
    // CTA's first loads then meet the bytes half way instead of starting HBM's latency from zero.
    for (int st = 0; st < num_stages && st < kRawStages; ++st) {
#pragma unroll
      for (int a = 0; a < kAtoms; ++a) tma_prefetch_l2_2d(&tmap_w, st * kStageK + a * 128, n0);
    }
  }
  if (warp == kMma) {
    tmem_alloc<1>(&tmem_base_slot, kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  griddep_wait();
  griddep_launch_dependents();

  auto stage_x = [&](int s) { return smem + kXOff + s * kXBytes; };
  auto stage_w = [&](int s) { return smem + kRawOff + s * kRawWBytes; };

  if (warp == kProducer) {
    if (lane == 0) {
      bool ok = true;
      for (int st = 0; st < num_stages && ok; ++st) {
        const int s = st % kRawStages, xs = st % kXStages;
        if (!mbar_wait(&raw_empty_bar[s], ((st / kRawStages) & 1) ^ 1, &abort_flag) ||
            !mbar_wait(&x_empty_bar[xs], ((st / kXStages) & 1) ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&raw_full_bar[s], static_cast<uint32_t>(p.cpc) * kStageK);  // (bytes past the end of a row arrive as zeros)
#pragma unroll
        for (int a = 0; a < kAtoms; ++a) {
          tma_load_2d(stage_w(s) + a * kAtomBytes, &tmap_w, &raw_full_bar[s], st * kStageK + a * 128, n0);
        }
        mbar_arrive_expect_tx(&x_full_bar[xs], kXBytes);
#pragma unroll
        for (int j = 0; j < kBlocksPerStage; ++j) {
          tma_load_2d(stage_x(xs) + j * kXAtomBytes, &tmap_x, &x_full_bar[xs], (st * kStageK + j * kBlockK) * 2, 0);
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
      }
    }
  } else if (warp >= kMma && warp < kMma + kMmaWarps) {
    if (lane == 0) {
      // Every tcgen05 issue costs the issuing thread some 90 cycles, sixteen of them per stage more
      // than the stage's bytes take to arrive: the blocks of a stage are dealt to four threads.
      const int mw = static_cast<int>(warp) - kMma;
      const uint32_t idesc = umma_idesc(kChannels, NTOK, 0u, 0u);
      const uint64_t xdesc0 = umma_desc_sw128(smem_u32(stage_x(0)));
      const uint32_t acc0 = tmem_base + mw * kChains * NTOK;
      uint32_t issued = 0;
      bool ok = true;
      for (int st = 0; st < num_stages && ok; ++st) {
        const int xs = st % kXStages, u = st % kUnits;
        if (!mbar_wait(&unit_full_bar[u], (st / kUnits) & 1, &abort_flag) ||
            !mbar_wait(&x_full_bar[xs], (st / kXStages) & 1, &abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int blocks = min(kBlocksPerStage, num_kb - st * kBlocksPerStage);
        const uint32_t a_tmem = tmem_base + kUnitCol0 + u * kUnitCols;
        for (int j = mw; j < blocks; j += kMmaWarps) {
          const uint64_t xd = xdesc0 + static_cast<uint64_t>((xs * kXBytes + j * kXAtomBytes) >> 4);
#pragma unroll
          for (int i = 0; i < 4; ++i) {  // 16 K positions: eight columns of the unit, 32 bytes of an x row
            umma_ts_f16(acc0 + (issued % kChains) * NTOK, a_tmem + (j * 4 + i) * 8, xd + i * 2, idesc, issued >= kChains ? 1u : 0u);
            ++issued;
          }
        }
        umma_commit(&unit_empty_bar[u]);
        umma_commit(&x_empty_bar[xs]);
      }
      if (ok) umma_commit(&acc_full_bar);
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
      }
    }
  } else if (warp < kProducer) {
    const uint32_t quarter = warp & 3;                       // the lanes of tensor memory this warp may touch
    const uint32_t group = warp >> 2;
    const uint32_t atom = group;                             // which 128 K positions of the stage
    const uint32_t row = quarter * 32 + lane;                // the channel this thread widens
    const uint32_t row_off = atom * kAtomBytes + row * 128, sw = row & 7;
    const uint32_t t_row = tmem_base + ((quarter * 32u) << 16) + kUnitCol0 + atom * (kUnitCols / kAtoms);
    bool ok = true;
    for (int st = 0; st < num_stages && ok; ++st) {
      const int s = st % kRawStages, u = st % kUnits;
      if (!mbar_wait(&raw_full_bar[s], (st / kRawStages) & 1, &abort_flag)) {
        ok = false;
        break;
      }
      // Read and widen into registers first, hand the raw stage back, and only then wait for the
      // unit (12.5 -> 12.2 us at sixteen rows).
      const uint8_t *raw = stage_w(s) + row_off;
      uint32_t w[4][16];
#pragma unroll
      for (uint32_t pp = 0; pp < 4; ++pp) {  // two 16-byte pieces -> 32 halves -> 16 columns
        const uint4 v0 = *reinterpret_cast<const uint4 *>(raw + (((2 * pp) ^ sw) << 4));
        const uint4 v1 = *reinterpret_cast<const uint4 *>(raw + (((2 * pp + 1) ^ sw) << 4));
        e4m3x4_to_f16x4(v0.x, &w[pp][0], &w[pp][1]);
        e4m3x4_to_f16x4(v0.y, &w[pp][2], &w[pp][3]);
        e4m3x4_to_f16x4(v0.z, &w[pp][4], &w[pp][5]);
        e4m3x4_to_f16x4(v0.w, &w[pp][6], &w[pp][7]);
        e4m3x4_to_f16x4(v1.x, &w[pp][8], &w[pp][9]);
        e4m3x4_to_f16x4(v1.y, &w[pp][10], &w[pp][11]);
        e4m3x4_to_f16x4(v1.z, &w[pp][12], &w[pp][13]);
        e4m3x4_to_f16x4(v1.w, &w[pp][14], &w[pp][15]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty_bar[s]);  // the raw bytes are in registers: the stage may be refilled
      if (!mbar_wait(&unit_empty_bar[u], ((st / kUnits) & 1) ^ 1, &abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();  // the instructions that read this unit last are done
#pragma unroll
      for (uint32_t pp = 0; pp < 4; ++pp) tmem_st_32x16(t_row + u * kUnitCols + pp * 16, w[pp]);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&unit_full_bar[u]);
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
    }
    // -------------------------------------------------------------- epilogue: the first four warps
    if (warp < 4 && __all_sync(0xffffffffu, ok)) {
      ok = mbar_wait(&acc_full_bar, 0, &abort_flag);
      if (__all_sync(0xffffffffu, ok)) {
        tc_fence_after_sync();
        const int local = static_cast<int>(warp) * 32 + static_cast<int>(lane);
        const int channel = n0 + local;
        const bool live = local < p.cpc && channel < p.n;
        const float scale = __ldg(p.scale);
        const float bias = (p.bias && live) ? __half2float(reinterpret_cast<const __half *>(p.bias)[channel]) : 0.0f;
        const __half *res = reinterpret_cast<const __half *>(p.residual);
        __half *out = reinterpret_cast<__half *>(p.out);
        for (int t0 = 0; t0 < NTOK && t0 < p.m; t0 += 16) {
          // the four partial sums of sixteen rows: all four loads, then one wait
          uint32_t v[16], u[kMmaWarps * kChains - 1][16];
          tmem_ld_32x16(tmem_base + ((warp * 32u) << 16) + t0, v);
#pragma unroll
          for (int c = 1; c < kMmaWarps * kChains; ++c) tmem_ld_32x16(tmem_base + ((warp * 32u) << 16) + c * NTOK + t0, u[c - 1]);
          tmem_ld_wait(v);
#pragma unroll
          for (int c = 1; c < kMmaWarps * kChains; ++c) {
            tmem_ld_wait(u[c - 1]);
            if (c / kChains < num_kb) {  // (an issuing warp beyond the last block of a short product wrote nothing)
#pragma unroll
              for (int t = 0; t < 16; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) + __uint_as_float(u[c - 1][t]));
            }
          }
          if (live) {
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              const int row = t0 + t;
              if (row < p.m) {
                float y = __uint_as_float(v[t]) * scale + bias;
                if (res) y += __half2float(res[static_cast<long long>(row % p.residual_rows) * p.residual_ld + channel]);
                out[static_cast<long long>(row) * p.n + channel] = __float2half_rn(y);
              }
            }
          }
        }
      } else if (lane == 0) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // copies that may still be in flight
    __syncthreads();
  }
  if (warp == kMma) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

// ---- e4m3 rows against an e4m3 weight (fl_fp8_linear's product after its quantiser) ------------
//
// Both operands are what tcgen05.mma kind::f8f6f4 multiplies, so nothing touches the weight
// between shared memory and the tensor core: the weight on the M side again (128 channels per
// CTA), up to 64 rows as N, K = 32 per instruction. A stage is 256 K positions: two 128-byte
// swizzle atoms of the weight (32 KB) and two of the rows (N x 128 bytes each); as many stages
// as fit (six for 16 rows, four for 64). Four threads issue two of a stage's eight instructions
// each into an accumulator of its own; warps 0-3 are the epilogue (a lane per channel): the
// four partial sums, then the tile kernel's arithmetic in its order: acc * (row scale * channel
// scale), + bias, GELU, + residual, one rounding.
namespace q8 {

constexpr int kMaxTokens = 64;
constexpr int kMaxStages = 6;
constexpr int kIssuers = 4;
constexpr int kQChains = 1;
constexpr int kQProducer = 4;
constexpr int kQMma = 5;
constexpr int kQThreads = (kQMma + kIssuers) * 32;
constexpr int kSmemLimit = 227 * 1024 - 1024;  // (static shared memory beside it)

struct QParams {
  const float *row_scale;
  const float *col_scale;
  int col_scale_scalar;
  const void *bias;
  const void *residual;
  int residual_rows;
  long long residual_ld;
  int act, is_bf16;
  void *out;
  int m, n, k;
  int kbytes;  // bytes of a row of either operand: k, or 2 k for 16-bit operands
  int ntok;    // N of the instruction: the rows rounded up to a multiple of 16
  int cpc;     // channels per CTA: at most 128, a multiple of 8
  int stages;
  uint32_t tmem_cols;
  uint32_t *status;
};

__device__ __forceinline__ float gelu_tanh_q(float x) {
  // x / (1 + 2^z), z = x (c0 + c1 x^2): the tile kernel's form of the tanh GELU, bit for bit.
  constexpr float kC0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  constexpr float kC1 = kC0 * 0.044715f;
  const float z = x * fmaf(x * x, kC1, kC0);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
  return x * r;
}

// KIND: kKindF8 (e4m3 codes on both sides), or kKindF16 / kKindBF16 for a 16-bit weight and 16-bit
// rows (fl_matmul's linear-layer case): the same bytes per stage, half the K positions, and
// nothing to scale.
template <int KIND>
__global__ void __launch_bounds__(kQThreads, 1)
fewrow_q8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const QParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t acc_full_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile uint32_t abort_flag;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * p.cpc;
  const int num_stages = (p.kbytes + kStageK - 1) / kStageK;  // a stage: 256 bytes of every row (the last may be part zeros)
  const int x_atom = p.ntok * 128;
  const int stage_bytes = kRawWBytes + kAtoms * x_atom;

  if (warp == 0) {
    if (static_cast<int>(lane) < p.stages) {
      mbar_init(&full_bar[lane], 1);
      mbar_init(&empty_bar[lane], kIssuers);
    }
    if (lane == 0) {
      abort_flag = 0;
      mbar_init(&acc_full_bar, kIssuers);
    }
    fence_barrier_init();
  }
  if (warp == kQProducer && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    // (the first stages of the weight into L2 ahead of the wait on the kernel before, as above)
    for (int st = 0; st < num_stages && st < p.stages; ++st) {
#pragma unroll
      for (int a = 0; a < kAtoms; ++a) tma_prefetch_l2_2d(&tmap_w, st * kStageK + a * 128, n0);
    }
  }
  if (warp == kQMma) {
    tmem_alloc<1>(&tmem_base_slot, p.tmem_cols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  griddep_wait();
  griddep_launch_dependents();

  if (warp == kQProducer) {
    if (lane == 0) {
      bool ok = true;
      for (int st = 0; st < num_stages && ok; ++st) {
        const int s = st % p.stages;
        if (!mbar_wait(&empty_bar[s], ((st / p.stages) & 1) ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        uint8_t *base = smem + s * stage_bytes;
        mbar_arrive_expect_tx(&full_bar[s], static_cast<uint32_t>(p.cpc * kStageK + kAtoms * x_atom));  // (bytes outside arrive as zeros)
#pragma unroll
        for (int a = 0; a < kAtoms; ++a) {
          tma_load_2d(base + a * kAtomBytes, &tmap_w, &full_bar[s], st * kStageK + a * 128, n0);
          tma_load_2d(base + kRawWBytes + a * x_atom, &tmap_x, &full_bar[s], st * kStageK + a * 128, 0);
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
      }
    }
  } else if (warp >= kQMma) {
    if (lane == 0) {
      const int mw = static_cast<int>(warp) - kQMma;
      constexpr uint32_t kFmt = KIND == kKindBF16 ? 1u : 0u;
      const uint32_t idesc = umma_idesc(kChannels, static_cast<uint32_t>(p.ntok), kFmt, kFmt);
      const uint32_t acc0 = tmem_base + mw * kQChains * p.ntok;
      // this thread's two instructions of a stage: 32-byte steps 2 mw and 2 mw + 1 of the eight
      const uint32_t atom = mw >> 1, step0 = (mw & 1) * 2;
      bool ok = true;
      for (int st = 0; st < num_stages && ok; ++st) {
        const int s = st % p.stages;
        if (!mbar_wait(&full_bar[s], (st / p.stages) & 1, &abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t base = smem_u32(smem + s * stage_bytes);
        const uint64_t wd = umma_desc_sw128(base + atom * kAtomBytes) + step0 * 2;
        const uint64_t xd = umma_desc_sw128(base + kRawWBytes + atom * x_atom) + step0 * 2;
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // this thread's two 32-byte steps of the stage
          umma_ss<KIND>(acc0 + (i % kQChains) * p.ntok, wd + i * 2, xd + i * 2, idesc, (st > 0 || i >= kQChains) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(&acc_full_bar);
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0-3)
    const bool ok = mbar_wait(&acc_full_bar, 0, &abort_flag);
    if (__all_sync(0xffffffffu, ok)) {
      tc_fence_after_sync();
      const int local = static_cast<int>(warp) * 32 + static_cast<int>(lane);
      const int channel = n0 + local;
      const bool live = local < p.cpc && channel < p.n;
      const float cs = p.col_scale ? __ldg(p.col_scale + (p.col_scale_scalar || !live ? 0 : channel)) : 1.0f;
      const uint16_t *bias16 = reinterpret_cast<const uint16_t *>(p.bias);
      float bias = 0.0f;
      if (bias16 && live) {
        const uint16_t b = bias16[channel];
        bias = p.is_bf16 ? __uint_as_float(static_cast<uint32_t>(b) << 16) : __half2float(__ushort_as_half(b));
      }
      const uint16_t *res = reinterpret_cast<const uint16_t *>(p.residual);
      uint16_t *out = reinterpret_cast<uint16_t *>(p.out);
      for (int t0 = 0; t0 < p.m; t0 += 16) {
        uint32_t v[16], u[kIssuers * kQChains - 1][16];
        tmem_ld_32x16(tmem_base + ((warp * 32u) << 16) + t0, v);
#pragma unroll
        for (int c = 1; c < kIssuers * kQChains; ++c) tmem_ld_32x16(tmem_base + ((warp * 32u) << 16) + c * p.ntok + t0, u[c - 1]);
        tmem_ld_wait(v);
#pragma unroll
        for (int c = 1; c < kIssuers * kQChains; ++c) {
          tmem_ld_wait(u[c - 1]);
#pragma unroll
          for (int t = 0; t < 16; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) + __uint_as_float(u[c - 1][t]));
        }
        if (live) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const int row = t0 + t;
            if (row < p.m) {
              const float rs = p.row_scale ? __ldg(p.row_scale + row) : 1.0f;
              float y = __uint_as_float(v[t]) * (rs * cs);
              if (bias16) y += bias;
              if (p.act == 1) y = gelu_tanh_q(y);
              if (res) {
                const uint16_t r16 = res[static_cast<long long>(row % p.residual_rows) * p.residual_ld + channel];
                y += p.is_bf16 ? __uint_as_float(static_cast<uint32_t>(r16) << 16) : __half2float(__ushort_as_half(r16));
              }
              out[static_cast<long long>(row) * p.n + channel] =
                  p.is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y)) : __half_as_ushort(__float2half_rn(y));
            }
          }
        }
      }
    } else if (lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // copies that may still be in flight
    __syncthreads();
  }
  if (warp == kQMma) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, p.tmem_cols);
  }
}

}  // namespace q8

// Channels per CTA. A CTA's time is its own chain over the k / 256 stages whatever the bytes a
// stage brings (112 channels on 147 CTAs measured the same as 128 on 128), so 128 unless that
// takes more than one round of the SMs: then the channels are dealt evenly over whole rounds
// (24576 x 12288: 65.2 us on 280 CTAs of 88 channels against 68.7 on 192 of 128).
int channels_per_cta(int n) {
  static const int sms = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v < 1) v = 148;
    return v;
  }();
  const int ctas128 = (n + kChannels - 1) / kChannels;
  if (ctas128 <= sms) return kChannels;
  const int target = (ctas128 + sms - 1) / sms * sms;
  const int cpc = ((n + target - 1) / target + 7) / 8 * 8;
  return cpc > kChannels ? kChannels : cpc;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      return reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

// A (rows, row_bytes) byte matrix read in boxes of box_bytes x box_rows, zeros outside.
bool make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes, uint32_t box_rows,
              CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool fewrow_tc_supported(int m, int n, int k, int is_bf16, const void *x, const void *w, const void *out) {
  if (is_bf16 || m < 1 || m > 4 * kTokens || n < 8 || n % 8 != 0 || k < kBlockK || k % kBlockK != 0) return false;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(out) & 1)) {
    return false;
  }
  return encode_fn() != nullptr;
}

cudaError_t fewrow_tc_matmul(const void *x, int m, int n, int k, const uint8_t *w, const float *scale, const void *bias,
                             const void *residual, int residual_rows, int64_t residual_ld, void *out, uint32_t *status,
                             cudaStream_t stream, const char **why) {
  *why = "";
  CUtensorMap tw, tx;
  const int ntok = m <= kTokens ? kTokens : m <= 2 * kTokens ? 2 * kTokens : 4 * kTokens;  // the instruction's N
  const int cpc = channels_per_cta(n);
  const bool w_ok = make_map(&tw, w, static_cast<uint64_t>(n), static_cast<uint64_t>(k), 128, static_cast<uint32_t>(cpc), CU_TENSOR_MAP_SWIZZLE_128B);
  if (!w_ok ||
      !make_map(&tx, x, static_cast<uint64_t>(m), static_cast<uint64_t>(k) * 2, kBlockK * 2, static_cast<uint32_t>(ntok),
                CU_TENSOR_MAP_SWIZZLE_128B)) {
    *why = "cuTensorMapEncodeTiled refused an operand";
    return cudaErrorInvalidValue;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fewrow_tc_kernel<kTokens>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TcCfg<kTokens>::kSmemBytes);
    if (e == cudaSuccess) {
      e = cudaFuncSetAttribute(fewrow_tc_kernel<2 * kTokens>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               TcCfg<2 * kTokens>::kSmemBytes);
    }
    if (e == cudaSuccess) {
      e = cudaFuncSetAttribute(fewrow_tc_kernel<4 * kTokens>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               TcCfg<4 * kTokens>::kSmemBytes);
    }
    if (e != cudaSuccess) {
      *why = "cudaFuncSetAttribute(max dynamic shared memory) failed";
      return e;
    }
    attr_set = true;
  }
  Params p = {};
  p.scale = scale;
  p.bias = bias;
  p.residual = residual;
  p.residual_rows = residual_rows > 0 ? residual_rows : 1;
  p.residual_ld = residual_ld;
  p.out = out;
  p.m = m;
  p.n = n;
  p.k = k;
  p.cpc = cpc;
  p.status = status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((n + cpc - 1) / cpc), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = ntok == kTokens       ? TcCfg<kTokens>::kSmemBytes
                         : ntok == 2 * kTokens ? TcCfg<2 * kTokens>::kSmemBytes
                                               : TcCfg<4 * kTokens>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = ntok == kTokens       ? cudaLaunchKernelEx(&cfg, fewrow_tc_kernel<kTokens>, tw, tx, p)
                  : ntok == 2 * kTokens ? cudaLaunchKernelEx(&cfg, fewrow_tc_kernel<2 * kTokens>, tw, tx, p)
                                        : cudaLaunchKernelEx(&cfg, fewrow_tc_kernel<4 * kTokens>, tw, tx, p);
  if (e != cudaSuccess) *why = "kernel launch failed";
  return e;
}

bool fewrow_q8_supported(int m, int n, int k, const void *codes, const void *w, const void *out) {
  if (m < 1 || m > q8::kMaxTokens || n < 8 || n % 8 != 0 || k < 16 || k % 16 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(out) & 1)) {
    return false;
  }
  return encode_fn() != nullptr;
}

namespace {

// elem: bytes per element of both operands (1: e4m3 codes, 2: half or bfloat16 as `is_bf16` says).
cudaError_t launch_q8(int elem, const void *rows, const float *row_scale, int m, int n, int k, const void *w,
                      const float *col_scale, int col_scale_scalar, const void *bias, const void *residual,
                      int residual_rows, int64_t residual_ld, int act, int is_bf16, void *out, uint32_t *status,
                      cudaStream_t stream, const char **why) {
  *why = "";
  const int ntok = (m + 15) / 16 * 16;
  const uint64_t kbytes = static_cast<uint64_t>(k) * elem;
  CUtensorMap tw, tx;
  const int cpc = channels_per_cta(n);
  if (!make_map(&tw, w, static_cast<uint64_t>(n), kbytes, 128, static_cast<uint32_t>(cpc), CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_map(&tx, rows, static_cast<uint64_t>(m), kbytes, 128, static_cast<uint32_t>(ntok), CU_TENSOR_MAP_SWIZZLE_128B)) {
    *why = "cuTensorMapEncodeTiled refused an operand";
    return cudaErrorInvalidValue;
  }
  const int stage_bytes = kRawWBytes + kAtoms * ntok * 128;
  int stages = q8::kSmemLimit / stage_bytes;
  if (stages > q8::kMaxStages) stages = q8::kMaxStages;
  const int smem_bytes = stages * stage_bytes + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(q8::fewrow_q8_kernel<kKindF8>, cudaFuncAttributeMaxDynamicSharedMemorySize, q8::kSmemLimit);
    if (e == cudaSuccess) {
      e = cudaFuncSetAttribute(q8::fewrow_q8_kernel<kKindF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, q8::kSmemLimit);
    }
    if (e == cudaSuccess) {
      e = cudaFuncSetAttribute(q8::fewrow_q8_kernel<kKindBF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, q8::kSmemLimit);
    }
    if (e != cudaSuccess) {
      *why = "cudaFuncSetAttribute(max dynamic shared memory) failed";
      return e;
    }
    attr_set = true;
  }
  q8::QParams p = {};
  p.row_scale = row_scale;
  p.col_scale = col_scale;
  p.col_scale_scalar = col_scale_scalar;
  p.bias = bias;
  p.residual = residual;
  p.residual_rows = residual_rows > 0 ? residual_rows : 1;
  p.residual_ld = residual_ld;
  p.act = act;
  p.is_bf16 = is_bf16;
  p.out = out;
  p.m = m;
  p.n = n;
  p.k = k;
  p.kbytes = static_cast<int>(kbytes);
  p.ntok = ntok;
  p.cpc = cpc;
  p.stages = stages;
  const int acc_cols = q8::kIssuers * q8::kQChains * ntok;
  p.tmem_cols = acc_cols <= 64 ? 64u : acc_cols <= 128 ? 128u : acc_cols <= 256 ? 256u : 512u;
  p.status = status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((n + cpc - 1) / cpc), 1, 1);
  cfg.blockDim = dim3(q8::kQThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = elem == 1   ? cudaLaunchKernelEx(&cfg, q8::fewrow_q8_kernel<kKindF8>, tw, tx, p)
                  : is_bf16   ? cudaLaunchKernelEx(&cfg, q8::fewrow_q8_kernel<kKindBF16>, tw, tx, p)
                              : cudaLaunchKernelEx(&cfg, q8::fewrow_q8_kernel<kKindF16>, tw, tx, p);
  if (e != cudaSuccess) *why = "kernel launch failed";
  return e;
}

}  // namespace

cudaError_t fewrow_q8_linear(const uint8_t *codes, const float *row_scale, int m, int n, int k, const uint8_t *w,
                             const float *col_scale, int col_scale_scalar, const void *bias, const void *residual,
                             int residual_rows, int64_t residual_ld, int act, int is_bf16, void *out, uint32_t *status,
                             cudaStream_t stream, const char **why) {
  return launch_q8(1, codes, row_scale, m, n, k, w, col_scale, col_scale_scalar, bias, residual, residual_rows, residual_ld,
                   act, is_bf16, out, status, stream, why);
}

bool fewrow_w16_supported(int m, int n, int k, const void *x, const void *w, const void *out) {
  if (m < 1 || m > q8::kMaxTokens || n < 8 || n % 8 != 0 || k < 8 || k % 8 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(out) & 1)) {
    return false;
  }
  return encode_fn() != nullptr;
}

cudaError_t fewrow_w16_matmul(const void *x, int is_bf16, int m, int n, int k, const void *w, const void *bias,
                              const void *residual, int residual_rows, int64_t residual_ld, void *out, uint32_t *status,
                              cudaStream_t stream, const char **why) {
  return launch_q8(2, x, nullptr, m, n, k, w, nullptr, 0, bias, residual, residual_rows, residual_ld, 0, is_bf16, out, status,
                   stream, why);
}

}  // namespace flsm100
