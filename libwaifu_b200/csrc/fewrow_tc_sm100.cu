// At most 16 activation rows against an e4m3 weight that is widened exactly to half (flint's
// fl_fp8_matmul, flint/cuda/gemm_fp8_cutlass.cu): a product bound by streaming the weight from HBM
// once. Here the weight sits on the M side of tcgen05.mma and the rows are its N = 16, so that no
// instruction of a CUDA core multiplies anything and the time does not depend on the row count
// (the kernel in skinny_sm100.cu, which multiplies on mma.sync, takes 20 us for one row against
// 16384 x 3072 and 36 us for sixteen; this one 17.4 us for either):
//   warp 4     producer: per stage of 256 K positions one TMA copy of 128 weight rows x 256 e4m3
//              bytes (as they lie) into a ring of two raw stages, and four copies of the 16 rows x
//              128 bytes of x (128-byte swizzle) into a ring of four; the weight is read exactly once;
//   warps 6-11 converters: widen a stage's weight bytes to half (cvt.rn.f16x2.e4m3x2, exact) into
//              four 128-row x 128-byte tiles in the 128-byte swizzle (two such sets), and hand the
//              raw stage back at once, so that its next load is on its way while the instructions
//              run (with the raw stage held until those were done the kernel took 21 us);
//   warp 5     one thread issues sixteen tcgen05.mma kind::f16 (M = 128 channels, N = 16 rows,
//              K = 16) per stage into four accumulators in turn (4 x 128 x 16 floats in tensor
//              memory); it waits and commits once per stage: every tcgen05 issue and every wait,
//              even on a completed barrier, costs the thread some 80 cycles or more, and with
//              hand-overs per 64 K positions the kernel took 25 us;
//   warps 0-3  epilogue: a lane owns a channel, reads its 4 x 16 partial sums and adds them; scale,
//              bias, residual, one rounding; for every row the warp stores 32 consecutive channels.
// A CTA owns 128 output channels and is paced by its own chain (load, widen, multiply) over the
// k / 256 stages, two of them in flight: 17 us at k = 3072 for any channel count, so the kernel is
// for wide weights. Every wait is bounded (status word, as everywhere else).
#include "fewrow_tc_sm100.cuh"

#include <cuda.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

constexpr int kChannels = 128;   // per CTA: the M of the instruction
constexpr int kTokens = 16;      // its N
constexpr int kBlockK = 64;      // K positions per block: 64 e4m3 bytes, 128 bytes of half, four instructions
constexpr int kBlocksPerStage = 4;
constexpr int kStageK = kBlocksPerStage * kBlockK;     // K positions per ring stage
constexpr int kRawWBytes = kChannels * kStageK;        // 32 KB
constexpr int kXAtomBytes = kTokens * kBlockK * 2;     // 2 KB: a block's 16 rows x 128 bytes
constexpr int kXBytes = kBlocksPerStage * kXAtomBytes; // 8 KB
constexpr int kStages = 2;                             // of raw weight bytes: given back as soon as they are widened
constexpr int kXStages = 4;                            // of x: given back when the instructions that read them are done
constexpr int kWideBytes = kChannels * kBlockK * 2;    // 16 KB
constexpr int kWideUnits = 2;                 // a unit: the four widened tiles of one stage
constexpr int kWide = kWideUnits * kBlocksPerStage;
constexpr int kChains = 4;                  // one accumulator per instruction of a block
constexpr int kAccCols = kChains * kTokens;  // 64 columns of tensor memory
constexpr int kProducerWarp = 4;
constexpr int kMmaWarp = 5;
constexpr int kConverterWarp0 = 6;
constexpr int kConverterWarps = 6;
constexpr int kThreads = (kConverterWarp0 + kConverterWarps) * 32;
constexpr int kWideOff = 0;                               // 1024-byte aligned tiles first
constexpr int kXOff = kWideOff + kWide * kWideBytes;      // then x's swizzled tiles
constexpr int kRingOff = kXOff + kXStages * kXBytes;      // then the raw weight stages
constexpr int kSmemBytes = kRingOff + kStages * kRawWBytes + 1024;
static_assert(kXBytes % 1024 == 0 && kWideBytes % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
static_assert(kSmemBytes <= 227 * 1024, "shared memory");

struct Params {
  const float *scale;
  const void *bias;
  const void *residual;
  int residual_rows;
  long long residual_ld;
  void *out;
  int m, n, k;
  uint32_t *status;
};

__global__ void __launch_bounds__(kThreads, 1)
fewrow_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t raw_full_bar[kStages], raw_empty_bar[kStages];
  __shared__ __align__(8) uint64_t x_full_bar[kXStages], x_empty_bar[kXStages];
  __shared__ __align__(8) uint64_t wide_full_bar[kWideUnits], wide_empty_bar[kWideUnits];
  __shared__ __align__(8) uint64_t acc_full_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile uint32_t abort_flag;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kChannels;
  const int num_kb = p.k / kBlockK;                                  // blocks
  const int num_stages = (num_kb + kBlocksPerStage - 1) / kBlocksPerStage;  // ring stages (the last may be part zeros)

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&raw_full_bar[s], 1);
      mbar_init(&raw_empty_bar[s], kConverterWarps);
    }
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(&x_full_bar[s], 1);
      mbar_init(&x_empty_bar[s], 1);
    }
    for (int w = 0; w < kWideUnits; ++w) {
      mbar_init(&wide_full_bar[w], kConverterWarps);
      mbar_init(&wide_empty_bar[w], 1);
    }
    mbar_init(&acc_full_bar, 1);
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == kMmaWarp) {
    tmem_alloc<1>(&tmem_base_slot, kAccCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  griddep_wait();
  griddep_launch_dependents();

  auto stage_x = [&](int s) { return smem + kXOff + s * kXBytes; };
  auto stage_w = [&](int s) { return smem + kRingOff + s * kRawWBytes; };
  auto wide = [&](int w) { return smem + kWideOff + w * kWideBytes; };

  if (warp == kProducerWarp) {
    if (lane == 0) {
      bool ok = true;
      for (int st = 0; st < num_stages && ok; ++st) {
        const int s = st % kStages, xs = st % kXStages;
        if (!mbar_wait(&raw_empty_bar[s], ((st / kStages) & 1) ^ 1, &abort_flag) ||
            !mbar_wait(&x_empty_bar[xs], ((st / kXStages) & 1) ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&raw_full_bar[s], kRawWBytes);  // (bytes past the end of a row arrive as zeros)
        tma_load_2d(stage_w(s), &tmap_w, &raw_full_bar[s], st * kStageK, n0);
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
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kChannels, kTokens, 0u, 0u);
      const uint64_t wdesc0 = umma_desc_sw128(smem_u32(wide(0)));
      const uint64_t xdesc0 = umma_desc_sw128(smem_u32(stage_x(0)));
      bool ok = true;
      // One wait and two commits per stage of four blocks: the thread's own instructions (each
      // tcgen05 issue, each wait on a completed barrier is some 80 cycles) are what a few-row
      // product has to keep off the path of the bytes.
      for (int st = 0; st < num_stages && ok; ++st) {
        const int xs = st % kXStages, u = st % kWideUnits;
        if (!mbar_wait(&wide_full_bar[u], (st / kWideUnits) & 1, &abort_flag) ||
            !mbar_wait(&x_full_bar[xs], (st / kXStages) & 1, &abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int blocks = min(kBlocksPerStage, num_kb - st * kBlocksPerStage);
        for (int j = 0; j < blocks; ++j) {
          const uint64_t wd = wdesc0 + static_cast<uint64_t>((u * kBlocksPerStage + j) * (kWideBytes >> 4));
          const uint64_t xd = xdesc0 + static_cast<uint64_t>((xs * kXBytes + j * kXAtomBytes) >> 4);
#pragma unroll
          for (int i = 0; i < kChains; ++i) {  // 16 K positions = 32 bytes of a row each
            umma_ss<kKindF16>(tmem_base + i * kTokens, wd + i * 2, xd + i * 2, idesc, (st > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit(&wide_empty_bar[u]);
        umma_commit(&x_empty_bar[xs]);
      }
      if (ok) umma_commit(&acc_full_bar);
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
      }
    }
  } else if (warp >= kConverterWarp0) {
    // 16 e4m3 bytes of a row -> 16 halves = two 16-byte pieces of the row's 128 bytes in the
    // 128-byte swizzle (piece index xor row % 8).
    const int cw = static_cast<int>(warp) - kConverterWarp0;
    bool ok = true;
    for (int st = 0; st < num_stages && ok; ++st) {
      const int s = st % kStages, u = st % kWideUnits;
      if (!mbar_wait(&raw_full_bar[s], (st / kStages) & 1, &abort_flag) ||
          !mbar_wait(&wide_empty_bar[u], ((st / kWideUnits) & 1) ^ 1, &abort_flag)) {
        ok = false;
        break;
      }
      const uint8_t *raw = stage_w(s);
      // a stage: 128 rows x 16 pieces of 16 e4m3 bytes; piece (r, c) belongs to block c / 4
#pragma unroll 4
      for (int piece = cw * 32 + static_cast<int>(lane); piece < kChannels * 16; piece += kConverterWarps * 32) {
        const uint32_t r = static_cast<uint32_t>(piece) >> 4, c = static_cast<uint32_t>(piece) & 15;
        const uint32_t j = c >> 2, q = c & 3;
        const uint4 v = *reinterpret_cast<const uint4 *>(raw + piece * 16);
        uint4 lo, hi;
        e4m3x4_to_f16x4(v.x, &lo.x, &lo.y);
        e4m3x4_to_f16x4(v.y, &lo.z, &lo.w);
        e4m3x4_to_f16x4(v.z, &hi.x, &hi.y);
        e4m3x4_to_f16x4(v.w, &hi.z, &hi.w);
        uint8_t *row_base = wide(u * kBlocksPerStage + j) + r * 128;
        *reinterpret_cast<uint4 *>(row_base + (((2 * q) ^ (r & 7)) << 4)) = lo;
        *reinterpret_cast<uint4 *>(row_base + (((2 * q + 1) ^ (r & 7)) << 4)) = hi;
      }
      fence_proxy_async_smem();  // the UMMA reads these bytes through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&raw_empty_bar[s]);  // the raw bytes have been read: the stage may be refilled at once
        mbar_arrive(&wide_full_bar[u]);
      }
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, kStatusFewRowTcTimeout);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const bool ok = mbar_wait(&acc_full_bar, 0, &abort_flag);
    if (__all_sync(0xffffffffu, ok)) {
      tc_fence_after_sync();
      uint32_t v[16];
      tmem_ld_32x16(tmem_base + ((warp * 32u) << 16), v);
      tmem_ld_wait(v);
#pragma unroll
      for (int c = 1; c < kChains; ++c) {
        uint32_t u[16];
        tmem_ld_32x16(tmem_base + ((warp * 32u) << 16) + c * kTokens, u);
        tmem_ld_wait(u);
#pragma unroll
        for (int t = 0; t < kTokens; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) + __uint_as_float(u[t]));
      }
      const int channel = n0 + static_cast<int>(warp) * 32 + static_cast<int>(lane);
      if (channel < p.n) {
        const float scale = __ldg(p.scale);
        const float bias = p.bias ? __half2float(reinterpret_cast<const __half *>(p.bias)[channel]) : 0.0f;
        const __half *res = reinterpret_cast<const __half *>(p.residual);
        __half *out = reinterpret_cast<__half *>(p.out);
#pragma unroll
        for (int t = 0; t < kTokens; ++t) {
          if (t < p.m) {
            float y = __uint_as_float(v[t]) * scale + bias;
            if (res) y += __half2float(res[static_cast<long long>(t % p.residual_rows) * p.residual_ld + channel]);
            out[static_cast<long long>(t) * p.n + channel] = __float2half_rn(y);
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
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kAccCols);
  }
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
  if (is_bf16 || m < 1 || m > kTokens || n < 8 || n % 8 != 0 || k < kBlockK || k % kBlockK != 0) return false;
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
  if (!make_map(&tw, w, static_cast<uint64_t>(n), static_cast<uint64_t>(k), kStageK, kChannels, CU_TENSOR_MAP_SWIZZLE_NONE) ||
      !make_map(&tx, x, static_cast<uint64_t>(m), static_cast<uint64_t>(k) * 2, kBlockK * 2, kTokens,
                CU_TENSOR_MAP_SWIZZLE_128B)) {
    *why = "cuTensorMapEncodeTiled refused an operand";
    return cudaErrorInvalidValue;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fewrow_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
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
  p.status = status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((n + kChannels - 1) / kChannels), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, fewrow_tc_kernel, tw, tx, p);
  if (e != cudaSuccess) *why = "kernel launch failed";
  return e;
}

}  // namespace flsm100
