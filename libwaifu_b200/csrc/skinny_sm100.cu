// The skinny case of the quantized linear: at most 16 activation rows (decode rows, the M = batch
// adaLN modulation and time-embedding linears, waifu/src/qwen_image/dit.rs:464-475,497-504,565).
// With so few rows the product is bound by streaming the weight from HBM once, so this kernel is
// shaped for bandwidth, not for the tensor pipe:
//
//   * one launch does everything, with no scratch: the CTA's eight consumer warps first put the
//     activation rows into shared memory, quantised per token to e4m3 codes with the same
//     arithmetic as quantize_fp8_act, while the producer warp is already streaming the weight;
//   * persistent CTAs, two per SM where the rows leave room (else one). The weight is (n, k)
//     row-major, so the K bytes of an
//     output channel are contiguous: the producer warp brings 8 x WN channels x up to 512 x WK
//     bytes per stage (WN x WK = 8) with one bulk copy (cp.async.bulk, no tensor map) per stage
//     or per channel into a ring of shared-memory stages that holds well over the
//     bandwidth-delay product of the SM;
//   * consumer warp (wn, wk) owns 8 channels and one K slice of each stage. With a quantised
//     activation the arithmetic is the warp-level mma.sync m16n8k32 e4m3 x e4m3 -> fp32 (exact
//     products, fp32 accumulation) straight from the bytes, no widening; the K order inside an
//     instruction is permuted so that a thread's 16 contiguous weight bytes feed two instructions
//     from one 16-byte shared-memory read, each into its own accumulator chain;
//   * with WK > 1 the partial sums of the K slices meet in shared memory once per unit of 8 x WN
//     channels, and the fused epilogue (row and channel scales, bias, GELU-tanh, residual, one
//     rounding) writes the 16-bit result. Its operands are staged in shared memory at the start.
//
// The same kernel serves the reference-compatible fl_fp8_matmul[_add], whose activation is not
// narrowed (flint/capi.cc:1011-1016): the rows go to shared memory as they are, the arithmetic is
// m16n8k16 on halves or bfloat16, and the weight's e4m3 bytes are widened in registers as the
// reference's kernel does (flint/cuda/gemm_fp8_cutlass.cu:20-29), with a few integer instructions
// (cvt makes the stream ALU-bound). This is the reference's decode shape (1 x 16384 x 3072,
// docs/fp8.md:225-244). And it serves the unquantised linear of fl_matmul[_add] (a 16-bit weight,
// no widening).
//
// Every wait on an mbarrier is bounded; a wait that gives up raises the CTA's abort flag, records
// a status code and the CTA leaves after a bounded wait for its copies in flight.
#include "skinny_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>
#include <cstdlib>

#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;  // + the producer warp
constexpr int kKStep = 64;                 // K bytes one warp consumes per step (two MMAs of 32)
constexpr int kWarpSlice = 512;            // K bytes of a stage one consumer warp owns (8 steps)
constexpr int kMaxStages = 5;
constexpr int kSmemBudget = 224 * 1024;
constexpr int kFixedSmem = 64 /*row scales*/ + 64 /*team amax*/ + 2 * kConsumerWarps * 128 * 4 /*partial sums*/ + 128 /*barriers*/;


__device__ __forceinline__ float widen16(uint16_t v, int is_bf16) {
  if (is_bf16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  return __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  constexpr float kC0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  constexpr float kC1 = kC0 * 0.044715f;
  const float z = x * fmaf(x * x, kC1, kC0);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
  return x * r;
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyParams {
  const uint16_t *x;  // (m, k) 16-bit
  int is_bf16;
  const uint8_t *w;   // (n, k) e4m3
  const float *col_scale;
  int col_scale_scalar;
  const void *bias;
  const void *residual;  // rows of n with pitch residual_ld, repeating with period residual_rows over m
  int residual_rows;
  long long residual_ld;
  int act;
  uint16_t *out;         // (m, n)
  int m, n, k;
  int kb;                // bytes of a weight row: k for e4m3, 2 k for a 16-bit weight
  int k_pad;             // every K position a step can touch, in elements (>= k)
  int pitch_x;           // bytes between activation rows in shared memory
  int x_vec;             // x is 16-byte aligned: 16-byte reads of the activation
  int out_pair;          // out is 4-byte aligned: two adjacent results go out as one store
  int wn_log2;           // WN = 1 << wn_log2 channel groups of 8 per unit; WK = 8 / WN K slices per stage
  int stages;            // ring depth
  int stage_stride;      // bytes of a ring stage
  int units;             // ceil(n / (8 WN))
  int k_chunks;          // stages per unit
  int chunk_bytes;       // K bytes of a full stage (a multiple of 64, at most 512 WK)
  int slice_bytes;       // K bytes of a stage one consumer warp owns (a multiple of 64, at most 512)
  int pitch_w;           // bytes between channels in a stage
  int one_copy;          // a stage is one contiguous piece of the weight (k_chunks == 1, pitch_w == k)
  int cpc;               // channels a CTA owns at most: ceil(units / grid) units of 8 WN
  int ep_bytes;          // shared memory of the staged epilogue operands
  uint32_t *status;
  int probe;             // development builds (-DFLSM100_PROBE) only
};

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

__device__ __forceinline__ float load16(const void *p, long long i, int is_bf16) {
  return widen16(__ldg(reinterpret_cast<const uint16_t *>(p) + i), is_bf16);
}

__device__ __forceinline__ uint32_t narrow16(float v, int is_bf16) {
  return is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

// Eight 16-bit elements of a row starting at element i (whole, by the k % 16 rule).
__device__ __forceinline__ uint4 load_x8(const uint16_t *src, int i, int x_vec) {
  if (x_vec) return __ldg(reinterpret_cast<const uint4 *>(src + i));
  uint16_t e[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) e[j] = __ldg(src + i + j);
  return make_uint4(e[0] | (uint32_t(e[1]) << 16), e[2] | (uint32_t(e[3]) << 16), e[4] | (uint32_t(e[5]) << 16),
                    e[6] | (uint32_t(e[7]) << 16));
}

// Largest magnitude among eight 16-bit elements.
__device__ __forceinline__ float amax8(const uint4 v, int is_bf16) {
  const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
  float a = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    a = fmaxf(a, fabsf(widen16(static_cast<uint16_t>(w4[j] & 0xffff), is_bf16)));
    a = fmaxf(a, fabsf(widen16(static_cast<uint16_t>(w4[j] >> 16), is_bf16)));
  }
  return a;
}

// Eight 16-bit elements -> the eight e4m3 codes of x * inv (round to nearest even, saturating).
__device__ __forceinline__ uint2 quantise8(const uint4 v, float inv, int is_bf16) {
  const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
  uint32_t two[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 pair = make_float2(__fmul_rn(widen16(static_cast<uint16_t>(w4[j] & 0xffff), is_bf16), inv),
                                    __fmul_rn(widen16(static_cast<uint16_t>(w4[j] >> 16), is_bf16), inv));
    two[j] = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(pair, __NV_SATFINITE, __NV_E4M3)) & 0xffff;
  }
  return make_uint2(two[0] | (two[1] << 16), two[2] | (two[3] << 16));
}

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four e4m3 bytes -> two registers of two 16-bit floats each, with integer instructions only (a
// cvt per pair would make the stream ALU-bound). A code S EEEE MMM placed as S 0EEEE MMM0000000
// is the half of value x 2^-8, subnormal codes included (both formats then have exponent field 0
// and the same fraction); the epilogue's scale carries the 2^8. For bfloat16 the same placement
// S 0000EEEE MMM0000 is value x 2^-120, and one bfloat16 multiplication by 2^120 makes it the
// value itself, exactly. The two NaN codes (0x7f, 0xff) come out as +-480: a weight holds none
// (the writers saturate to +-448, tools/model_writer.py:162-170).
template <bool BF16>
__device__ __forceinline__ void widen_e4m3x4(uint32_t w, uint32_t &p01, uint32_t &p23) {
  uint32_t hi, lo;
  if constexpr (!BF16) {
    hi = ((w >> 1) & 0x3f3f3f3fu) | (w & 0x80808080u);  // S 0 E E E E M M of every byte
    lo = (w << 7) & 0x80808080u;                         // M 0 0 0 0 0 0 0
  } else {
    hi = ((w >> 4) & 0x07070707u) | (w & 0x80808080u);  // S 0 0 0 0 E E E
    lo = (w << 4) & 0xf0f0f0f0u;                         // E M M M 0 0 0 0
  }
  p01 = __byte_perm(lo, hi, 0x5140);
  p23 = __byte_perm(lo, hi, 0x7362);
  if constexpr (BF16) {
    const uint32_t two120 = 0x7b807b80u;  // 2^120 twice
    const __nv_bfloat162 k = *reinterpret_cast<const __nv_bfloat162 *>(&two120);
    __nv_bfloat162 a = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&p01), k);
    __nv_bfloat162 b = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&p23), k);
    p01 = *reinterpret_cast<const uint32_t *>(&a);
    p23 = *reinterpret_cast<const uint32_t *>(&b);
  }
}

// QUANT: the activation rows are quantised per token to e4m3 first, kept as codes and multiplied
// on the FP8 form of mma.sync; else they stay 16-bit. BF16: the 16-bit product runs on bfloat16
// instructions (never with QUANT).
// W16: the weight itself is 16-bit (the unquantised linear layer of fl_matmul): no widening, eight
// K positions per 16-byte piece instead of sixteen.
template <bool QUANT, bool BF16, bool W16>
__global__ void __launch_bounds__(kThreads, 2) skinny_fp8_kernel(const SkinnyParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int x_bytes = (p.m * p.pitch_x + 127) / 128 * 128;
  uint8_t *xq = smem;                                               // [m][pitch_x]
  float *row_scale = reinterpret_cast<float *>(smem + x_bytes);     // [16]
  float *team_amax = row_scale + 16;                                // [16]
  float *red = team_amax + 16;                                      // [2][8 warps][32 lanes][4]
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(red + 2 * kConsumerWarps * 128);  // [kMaxStages]
  uint64_t *empty_bar = full_bar + kMaxStages;                      // [kMaxStages]
  // Epilogue operands of all the channels this CTA owns, fetched once at the start: a unit can be
  // a single stage long, far shorter than a trip to global memory.
  float *cs_s = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(full_bar) + 128);  // [cpc] channel scales
  float *bias_s = cs_s + p.cpc;                                                           // [cpc]
  uint16_t *res_s = reinterpret_cast<uint16_t *>(bias_s + p.cpc);                         // [m][cpc], if any
  uint8_t *ring = reinterpret_cast<uint8_t *>(cs_s) + p.ep_bytes;   // [stages][stage_stride]
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int WN = 1 << p.wn_log2;
  const int WK = kConsumerWarps >> p.wn_log2;
  const int unit_rows = 8 * WN;
  const int chunk_bytes = p.chunk_bytes;
  const int pitch_w = p.pitch_w;  // 64 mod 128: a quarter warp's 16-byte reads of two rows miss each other

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    fence_barrier_init();
  }
  __syncthreads();
  griddep_wait();
  griddep_launch_dependents();

  if (warp == kConsumerWarps) {
    // ================= producer: one bulk copy per channel and stage =================
    int stage = 0;
    uint32_t phase = 0;
    uint32_t armed = 0;  // stages whose full barrier has been armed at least once (bit s)
    bool ok = true;
#ifdef FLSM100_PROBE
    long long probe_wait = 0;
    const long long probe_start = clock64();
#endif
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      const int row0 = u * unit_rows;
      const int rows = min(unit_rows, p.n - row0);
      for (int kc = 0; kc < p.k_chunks; ++kc) {
        int got = 1;
#ifdef FLSM100_PROBE
        const long long pw0 = clock64();
#endif
        if (lane == 0) got = mbar_wait(&empty_bar[stage], phase ^ 1, &abort_flag) ? 1 : 0;
#ifdef FLSM100_PROBE
        probe_wait += clock64() - pw0;
#endif
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          ok = false;
          break;
        }
        const int k0 = kc * chunk_bytes;
        const uint32_t bytes = static_cast<uint32_t>(min(chunk_bytes, p.kb - k0));
        if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], bytes * rows);
        __syncwarp();
        uint8_t *dst = ring + stage * p.stage_stride;
        if (p.one_copy) {
          // A stage holds whole channels, which are contiguous in the weight: one copy for all.
          if (lane == 0) bulk_load_1d(dst, p.w + static_cast<long long>(row0) * p.kb, bytes * rows, &full_bar[stage]);
        } else {
          for (int r = lane; r < rows; r += 32) {
            bulk_load_1d(dst + r * pitch_w, p.w + static_cast<long long>(row0 + r) * p.kb + k0, bytes, &full_bar[stage]);
          }
        }
        armed |= 1u << stage;
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusProducerTimeout));
    }
#ifdef FLSM100_PROBE
    if ((p.probe & 16) && blockIdx.x == 0 && lane == 0)
      printf("producer: %lld cycles, %lld waiting for empty stages\n", clock64() - probe_start, probe_wait);
#endif
    // Leave only when no copy of this CTA is still in flight. After a normal run the consumers
    // have waited for every stage already and these waits return at once.
    if (lane == 0) {
      volatile uint32_t never = 0;
      for (int s = 0; s < p.stages; ++s) {
        if (!(armed & (1u << s))) continue;
        // The last phase armed on stage s: the current one if the ring position has passed s in
        // this round, the previous one otherwise.
        const uint32_t last = (s < stage) ? phase : (phase ^ 1);
        mbar_wait(&full_bar[s], last, &never);
      }
    }
    return;
  }

  // ================= consumers =================
#ifdef FLSM100_PROBE
  const long long probe_start = clock64();
  long long probe_wait = 0, probe_prologue = 0;
#endif
  constexpr float kUnfoldStage = (BF16 || W16 || QUANT) ? 1.0f : 256.0f;  // see kUnfold below
  // ---- 0. this CTA's channel scales and bias: issued now, stored after the activation rows
  const bool vector_scale = p.col_scale && !p.col_scale_scalar;
  auto channel_of = [&](int i) {  // i = local unit * unit_rows + channel in unit; -1 when there is none
    const int j = i / unit_rows;
    const int u = blockIdx.x + j * gridDim.x;
    const int ch = u * unit_rows + (i - j * unit_rows);
    return (u < p.units && ch < p.n) ? ch : -1;
  };
  float first_cs = 1.0f, first_bias = 0.0f;
  {
    const int ch = threadIdx.x < p.cpc ? channel_of(threadIdx.x) : -1;
    if (ch >= 0) {
      if (vector_scale) first_cs = __ldg(p.col_scale + ch);
      if (p.bias) first_bias = load16(p.bias, ch, p.is_bf16);
    }
  }

  // ---- 1. the activation rows into shared memory
  if constexpr (QUANT) {
    // T warps share a row so that a single row still uses the whole CTA.
    const int T = p.m == 1 ? 8 : p.m == 2 ? 4 : p.m <= 4 ? 2 : 1;
    const int rows_per_round = kConsumerWarps / T;
    const int tw = warp % T;
    for (int r0 = 0; r0 < p.m; r0 += rows_per_round) {  // one round whenever T > 1
      const int r = r0 + warp / T;
      const bool active = r < p.m;
      const uint16_t *src = p.x + static_cast<long long>(active ? r : 0) * p.k;
      // The first two pieces a thread reads stay in registers for the second pass (all of the
      // row up to k = 4096 T); longer rows read the rest again.
      const int i0 = (tw * 32 + lane) * 8;
      const int stride = T * 256;
      const uint4 zero = make_uint4(0, 0, 0, 0);
      uint4 keep0 = zero, keep1 = zero;
      float amax = 0.0f;
      if (active) {
        if (i0 < p.k) keep0 = load_x8(src, i0, p.x_vec);
        if (i0 + stride < p.k) keep1 = load_x8(src, i0 + stride, p.x_vec);
        amax = fmaxf(amax8(keep0, p.is_bf16), amax8(keep1, p.is_bf16));
#pragma unroll 4
        for (int i = i0 + 2 * stride; i < p.k; i += stride) amax = fmaxf(amax, amax8(load_x8(src, i, p.x_vec), p.is_bf16));
      }
      amax = warp_max(amax);
      if (T > 1) {
        if (lane == 0) team_amax[warp] = amax;
        consumer_barrier();
        for (int j = 0; j < T; ++j) amax = fmaxf(amax, team_amax[warp / T * T + j]);
      }
      if (!active) continue;
      const float scale = __fdiv_rn(amax, 448.0f);
      const float inv = __frcp_rn(scale > 0.0f ? scale : 1.0f);
      if (lane == 0 && tw == 0) row_scale[r] = scale;
      uint8_t *dst = xq + r * p.pitch_x;
      // zeros past k (a group of 8 is whole or absent)
      const uint2 none = make_uint2(0, 0);
      if (i0 < p.k_pad) *reinterpret_cast<uint2 *>(dst + i0) = i0 < p.k ? quantise8(keep0, inv, p.is_bf16) : none;
      if (i0 + stride < p.k_pad) {
        *reinterpret_cast<uint2 *>(dst + i0 + stride) = i0 + stride < p.k ? quantise8(keep1, inv, p.is_bf16) : none;
      }
#pragma unroll 4
      for (int i = i0 + 2 * stride; i < p.k_pad; i += stride) {
        *reinterpret_cast<uint2 *>(dst + i) = i < p.k ? quantise8(load_x8(src, i, p.x_vec), inv, p.is_bf16) : none;
      }
    }
  } else {
    const int groups = p.k_pad / 8;  // 16-byte groups per row
#pragma unroll 4
    for (int idx = threadIdx.x; idx < p.m * groups; idx += kConsumers) {
      const int r = idx / groups;
      const int i = (idx - r * groups) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (i < p.k) v = load_x8(p.x + static_cast<long long>(r) * p.k, i, p.x_vec);
      *reinterpret_cast<uint4 *>(xq + r * p.pitch_x + 2 * i) = v;
    }
  }
  if (threadIdx.x < p.cpc) {
    cs_s[threadIdx.x] = first_cs * kUnfoldStage;
    bias_s[threadIdx.x] = first_bias;
  }
  for (int i = threadIdx.x + kConsumers; i < p.cpc; i += kConsumers) {
    const int ch = channel_of(i);
    cs_s[i] = ((ch >= 0 && vector_scale) ? __ldg(p.col_scale + ch) : 1.0f) * kUnfoldStage;
    bias_s[i] = (ch >= 0 && p.bias) ? load16(p.bias, ch, p.is_bf16) : 0.0f;
  }
  if (p.residual) {
#pragma unroll 4
    for (int idx = threadIdx.x; idx < p.m * p.cpc; idx += kConsumers) {
      const int r = idx / p.cpc;
      const int ch = channel_of(idx - r * p.cpc);
      res_s[idx] = ch >= 0 ? __ldg(reinterpret_cast<const uint16_t *>(p.residual) +
                                   static_cast<long long>(r % p.residual_rows) * p.residual_ld + ch)
                           : uint16_t(0);
    }
  }
  consumer_barrier();
#ifdef FLSM100_PROBE
  probe_prologue = clock64() - probe_start;
#endif

  // ---- 2. the weight stream
  const int wn = warp / WK;
  const int wk = warp - wn * WK;
  const int g = lane >> 2;  // row of the A fragment / channel of the B fragment
  const int q = lane & 3;   // which 16 of a step's 64 K bytes this thread holds
  const bool row_lo = g < p.m;
  const bool row_hi = g + 8 < p.m;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  // The half path multiplies weight values scaled by 2^-8; the scale gives the 2^8 back (exactly).
  constexpr float kUnfold = (BF16 || W16 || QUANT) ? 1.0f : 256.0f;
  const float scalar_scale = ((p.col_scale && p.col_scale_scalar) ? __ldg(p.col_scale) : 1.0f) * kUnfold;

  int stage = 0;
  uint32_t phase = 0;
  uint32_t unit_parity = 0;
  bool ok = true;
  int local_unit = 0;
  for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, unit_parity ^= 1, ++local_unit) {
    const int n_first = u * unit_rows + wn * 8;  // this warp's 8 channels
    const int nc = n_first + 2 * q;              // this thread's two result channels
    const bool writer = wk == 0 && n_first < p.n;
    // Eight accumulator chains: the four instructions of a step and those of the next step all go
    // to different ones, so that no instruction waits for the one before it.
    constexpr int kSteps = kWarpSlice / kKStep;
    float acc[8][4];
#pragma unroll
    for (int s = 0; s < 8; ++s) acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.0f;
    const int steps = p.slice_bytes / kKStep;

    for (int kc = 0; kc < p.k_chunks; ++kc) {
#ifdef FLSM100_PROBE
      const long long cw0 = clock64();
#endif
      if (!mbar_wait(&full_bar[stage], phase, &abort_flag)) {
        ok = false;
        break;
      }
#ifdef FLSM100_PROBE
      probe_wait += clock64() - cw0;
      if (p.probe & 1) {  // timing probe: release the stage unread
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
        continue;
      }
#endif
#ifdef FLSM100_PROBE
      if (p.probe & 2) {  // timing probe: one shared-memory read per thread instead of the arithmetic
        acc[0][0] += *reinterpret_cast<const float *>(ring + stage * p.stage_stride + threadIdx.x * 4);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
        continue;
      }
#endif
      // No piece is predicated: past k the activation rows hold zeros, and the weight bytes read
      // there (stale, but finite once widened) multiply them; rows past m read row 0 and their
      // sums are never stored.
      const int kb0 = kc * chunk_bytes + wk * p.slice_bytes + q * 16;  // this thread's K byte in step 0
      const uint8_t *wrow = ring + stage * p.stage_stride + (wn * 8 + g) * pitch_w + wk * p.slice_bytes + q * 16;
      // the activation's byte offset for weight byte kb0: two bytes per e4m3 byte, one per byte of a 16-bit weight
      const int xoff = (W16 || QUANT) ? kb0 : 2 * kb0;  // QUANT keeps the rows as e4m3 codes, one byte each
      const uint8_t *xlo = xq + (row_lo ? g : 0) * p.pitch_x + xoff;
      const uint8_t *xhi = xq + (row_hi ? g + 8 : 0) * p.pitch_x + xoff;
#pragma unroll
      for (int s = 0; s < kSteps; ++s) {
        if (s < steps) {
          uint4 wv = *reinterpret_cast<const uint4 *>(wrow + s * kKStep);
          if constexpr (QUANT) {
            // e4m3 x e4m3 on the FP8 form of the instruction: no widening at all. A stale byte past
            // the end of the row may be a NaN code, which would not multiply a zero to zero.
            if (kb0 + s * kKStep >= min(p.kb, (kc + 1) * chunk_bytes)) wv = zero4;
            const uint4 xa = *reinterpret_cast<const uint4 *>(xlo + s * kKStep);
            uint4 xb = zero4;
            if (p.m > 8) xb = *reinterpret_cast<const uint4 *>(xhi + s * kKStep);
            // Logical k of an instruction <-> physical byte: registers (x, y) of the 16 bytes are
            // the "low" and "high" halves of the first instruction, (z, w) of the second; the same
            // permutation on both operands, so every product pairs the same physical k.
            mma_e4m3(acc[((s & 3) << 1)], xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
            mma_e4m3(acc[((s & 3) << 1) | 1], xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
          } else if constexpr (W16) {
            // Past the end of the row the stage holds stale bytes, which as 16-bit floats may be
            // NaN or infinite and would not multiply the activation's zeros to zero.
            if (kb0 + s * kKStep >= min(p.kb, (kc + 1) * chunk_bytes)) wv = zero4;
            // 8 elements of row g (and g + 8) for this thread's 8 K positions; instruction i takes
            // positions 4i..4i+3, the first pair its "low" half, the second its "high" half.
            const uint4 xa = *reinterpret_cast<const uint4 *>(xlo + s * kKStep);
            uint4 xb = zero4;
            if (p.m > 8) xb = *reinterpret_cast<const uint4 *>(xhi + s * kKStep);
            float(&c0)[4] = acc[((s & 3) << 1)];
            float(&c1)[4] = acc[((s & 3) << 1) | 1];
            if constexpr (BF16) {
              mma_bf16(c0, xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
              mma_bf16(c1, xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
            } else {
              mma_f16(c0, xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
              mma_f16(c1, xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
            }
          } else {
            // 16 elements of row g (and g + 8) for this thread's 16 K positions.
            const uint4 xa0 = *reinterpret_cast<const uint4 *>(xlo + 2 * s * kKStep);
            const uint4 xa1 = *reinterpret_cast<const uint4 *>(xlo + 2 * s * kKStep + 16);
            uint4 xb0 = zero4, xb1 = zero4;
            if (p.m > 8) {
              xb0 = *reinterpret_cast<const uint4 *>(xhi + 2 * s * kKStep);
              xb1 = *reinterpret_cast<const uint4 *>(xhi + 2 * s * kKStep + 16);
            }
            const uint32_t al[8] = {xa0.x, xa0.y, xa0.z, xa0.w, xa1.x, xa1.y, xa1.z, xa1.w};
            const uint32_t ah[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
            const uint32_t wb[4] = {wv.x, wv.y, wv.z, wv.w};
            // Instruction i takes K positions 4i..4i+3 of the thread's 16: the first pair is its
            // "low" half and the second its "high" half, for A and for B alike, so every product
            // pairs the same physical k whatever order the instruction gives them.
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t w0, w1;
              widen_e4m3x4<BF16>(wb[i], w0, w1);
              float(&chain)[4] = acc[((s & 1) << 2) | i];
              if constexpr (BF16) mma_bf16(chain, al[2 * i], ah[2 * i], al[2 * i + 1], ah[2 * i + 1], w0, w1);
              else mma_f16(chain, al[2 * i], ah[2 * i], al[2 * i + 1], ah[2 * i + 1], w0, w1);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == p.stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (!ok) break;

    // ---- 3. the K slices of a channel group meet in shared memory
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = ((acc[0][i] + acc[1][i]) + (acc[2][i] + acc[3][i])) + ((acc[4][i] + acc[5][i]) + (acc[6][i] + acc[7][i]));
    }
#ifdef FLSM100_PROBE
    if (p.probe & 4) continue;  // timing probe: no reduction, no epilogue
#endif
    if (WK > 1) {
      float4 *buf = reinterpret_cast<float4 *>(red + unit_parity * kConsumerWarps * 128);
      if (wk != 0) buf[warp * 32 + lane] = make_float4(v[0], v[1], v[2], v[3]);
      consumer_barrier();  // the buffer of this parity is written again two units later, after the next barrier
      if (wk == 0) {
        for (int j = 1; j < WK; ++j) {
          const float4 o = buf[(warp + j) * 32 + lane];
          v[0] += o.x;
          v[1] += o.y;
          v[2] += o.z;
          v[3] += o.w;
        }
      }
    }

    // ---- 4. fused epilogue: v[0], v[1] are row g, v[2], v[3] row g + 8, channels nc and nc + 1
    if (writer) {
      const int e = local_unit * unit_rows + wn * 8 + 2 * q;  // this thread's first channel among the CTA's
      const float cs0 = vector_scale ? cs_s[e] : scalar_scale, cs1 = vector_scale ? cs_s[e + 1] : scalar_scale;
      const float b0 = bias_s[e], b1 = bias_s[e + 1];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h;
        if (r >= p.m) continue;
        const float rs = QUANT ? row_scale[r] : 1.0f;
        float y0 = v[2 * h] * (rs * cs0) + b0;
        float y1 = v[2 * h + 1] * (rs * cs1) + b1;
        if (p.act == 1) {
          y0 = gelu_tanh(y0);
          y1 = gelu_tanh(y1);
        }
        if (p.residual) {
          y0 += widen16(res_s[r * p.cpc + e], p.is_bf16);
          y1 += widen16(res_s[r * p.cpc + e + 1], p.is_bf16);
        }
        uint16_t *o = p.out + static_cast<long long>(r) * p.n + nc;
        const uint32_t lo = narrow16(y0, p.is_bf16), hi = narrow16(y1, p.is_bf16);
        if (p.out_pair) {
          *reinterpret_cast<uint32_t *>(o) = lo | (hi << 16);
        } else {
          o[0] = static_cast<uint16_t>(lo);
          o[1] = static_cast<uint16_t>(hi);
        }
      }
    }
  }
  if (!ok && lane == 0) {
    abort_flag = 1;
    atomicCAS(p.status, 0u, static_cast<uint32_t>(kStatusEpilogueTimeout));
  }
#ifdef FLSM100_PROBE
  if ((p.probe & 16) && blockIdx.x == 0 && threadIdx.x == 0)
    printf("consumer warp 0: %lld cycles, prologue %lld, waiting for full stages %lld\n", clock64() - probe_start,
           probe_prologue, probe_wait);
#endif
}

int sm_count_cached() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

// K split: WK warps share a stage's K bytes; K goes in equal chunks of at most 512 WK bytes, a
// chunk in WK equal slices of whole steps, so that every warp is busy and every stage carries the
// same load. k_pad is every K position a step can touch: the activation rows are zero from k up
// to there, and whatever the weight's stage holds there multiplies zero.
struct KSplit {
  int k_chunks, chunk_bytes, slice_bytes, k_pad;
};

KSplit k_split(int k, int wn_log2) {
  const int wk = kConsumerWarps >> wn_log2;
  KSplit s;
  // A chunk is WK whole slices and a slice whole steps, so that the slices of a full chunk end
  // where the chunk ends: a read past the end of a chunk can only happen in the last one, past k.
  const int chunks = (k + kWarpSlice * wk - 1) / (kWarpSlice * wk);
  s.chunk_bytes = ((k + chunks - 1) / chunks + kKStep * wk - 1) / (kKStep * wk) * (kKStep * wk);
  s.slice_bytes = s.chunk_bytes / wk;
  s.k_chunks = (k + s.chunk_bytes - 1) / s.chunk_bytes;
  s.k_pad = s.k_chunks * s.chunk_bytes;
  return s;
}

// Bytes between the activation rows in shared memory, chosen so that the 16-byte reads a quarter
// warp makes of two rows fall into distinct banks: 16 mod 32 for 16-bit rows (pieces 32 bytes
// apart), 64 mod 128 for rows of e4m3 codes.
int row_pitch(int k_pad_elements, int xbytes) {
  if (xbytes == 2) return 2 * k_pad_elements + 16;
  // e4m3 rows: four 16-byte pieces per row and step, so 64 mod 128
  return k_pad_elements + (k_pad_elements % 128 == 0 ? 64 : 0);
}

inline int wk_of(int wn_log2) { return kConsumerWarps >> wn_log2; }

struct Geometry {
  int ctas, wn_log2, units, grid, cpc, ep_bytes, x_bytes, stages, stage_stride, pitch_w, one_copy;
  KSplit ks;
};

int pick_wn_log2(int k);

// Shared-memory plan of one CTA when `ctas` CTAs share an SM.
Geometry geometry_with(int m, int n, int k, int wbytes, int xbytes, bool has_residual, int ctas) {
  Geometry g;
  g.ctas = ctas;
  const int kb = k * wbytes;  // bytes of a weight row
  g.wn_log2 = pick_wn_log2(kb);
  const int rows = 8 << g.wn_log2;
  const int slots = sm_count_cached() * ctas;
  g.units = (n + rows - 1) / rows;
  g.grid = g.units < slots ? g.units : slots;
  g.cpc = (g.units + g.grid - 1) / g.grid * rows;
  g.ep_bytes = (g.cpc * 8 + (has_residual ? m * g.cpc * 2 : 0) + 127) / 128 * 128;
  g.ks = k_split(kb, g.wn_log2);
  g.x_bytes = (m * row_pitch(g.ks.k_pad / wbytes, xbytes) + 127) / 128 * 128;
  // With all of K in one stage the channels of a stage are one contiguous piece of the weight and
  // a single large copy brings them; the price is a two-way bank conflict on the weight reads
  // when k is a multiple of 128, far from what limits the kernel. Otherwise a channel's piece is
  // padded to 64 mod 128 bytes so that the reads of two channels miss each other.
  g.one_copy = g.ks.k_chunks == 1 ? 1 : 0;
  // The warps of a stage read WK whole slices of every channel, which can reach past the bytes a
  // chunk carries (the slices are whole steps): the pitch covers that reach, and where the pitch is
  // the row itself (one copy) the stage ends that much after its last channel, so that every read
  // stays inside the stage.
  const int reach = wk_of(g.wn_log2) * g.ks.slice_bytes;
  const int span = reach > g.ks.chunk_bytes ? reach : g.ks.chunk_bytes;
  g.pitch_w = g.one_copy ? kb : (span + 127) / 128 * 128 + 64;
  const int last = g.pitch_w > reach ? g.pitch_w : reach;
  g.stage_stride = ((rows - 1) * g.pitch_w + last + 127) / 128 * 128;
  const long long budget = kSmemBudget / ctas - (ctas > 1 ? 1024 : 0);  // less the per-CTA reserve
  const long long left = budget - kFixedSmem - g.x_bytes - g.ep_bytes;
  g.stages = left < 0 ? 0 : (left / g.stage_stride > kMaxStages ? kMaxStages : static_cast<int>(left / g.stage_stride));
  return g;
}

// The consumers are bound by instruction latency, not by issue slots, so two CTAs per SM (twice
// the warps, half the shared memory each) stream faster than one; a shape whose activation rows
// leave a half too small for three stages gets one CTA per SM.
Geometry geometry_for(int m, int n, int k, int wbytes, int xbytes, bool has_residual) {
  const Geometry two = geometry_with(m, n, k, wbytes, xbytes, has_residual, 2);
  return two.stages >= 3 ? two : geometry_with(m, n, k, wbytes, xbytes, has_residual, 1);
}

// Channel groups per unit. A channel's K bytes arrive as one bulk copy per stage, and long copies
// stream best, so K is split over as many warps as it has 512-byte slices (WK = 1, 2, 4 or 8) and
// the remaining warps take further channel groups (WN = 8 / WK).
int pick_wn_log2(int k) {
  const int slices = (k + kWarpSlice - 1) / kWarpSlice;
  return slices >= 5 ? 0 : slices >= 3 ? 1 : slices == 2 ? 2 : 3;
}

template <bool QUANT, bool BF16, bool W16>
cudaError_t launch(SkinnyParams &p, cudaStream_t stream) {
  constexpr int wbytes = W16 ? 2 : 1;
  constexpr int xbytes = QUANT ? 1 : 2;
  p.kb = p.k * wbytes;
  p.x_vec = (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 ? 1 : 0;
  p.out_pair = (reinterpret_cast<uintptr_t>(p.out) & 3) == 0 ? 1 : 0;
  const Geometry geo = geometry_for(p.m, p.n, p.k, wbytes, xbytes, p.residual != nullptr);
  p.wn_log2 = geo.wn_log2;
  p.stages = geo.stages;
  p.units = geo.units;
  p.cpc = geo.cpc;
  p.ep_bytes = geo.ep_bytes;
  p.stage_stride = geo.stage_stride;
  p.k_chunks = geo.ks.k_chunks;
  p.chunk_bytes = geo.ks.chunk_bytes;
  p.slice_bytes = geo.ks.slice_bytes;
  p.k_pad = geo.ks.k_pad / wbytes;
  p.pitch_x = row_pitch(p.k_pad, xbytes);
  p.pitch_w = geo.pitch_w;
  p.one_copy = geo.one_copy;
  const size_t smem = static_cast<size_t>(geo.x_bytes) + kFixedSmem + geo.ep_bytes + static_cast<size_t>(p.stages) * geo.stage_stride;

  p.probe = 0;
#ifdef FLSM100_PROBE
  if (const char *v = std::getenv("FLSM100_PROBE")) p.probe = std::atoi(v);
#endif
  auto kernel = skinny_fp8_kernel<QUANT, BF16, W16>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(geo.grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

bool supported(int m, int n, int k, int wbytes, int xbytes, const void *x, const void *w, const void *out, bool has_residual) {
  if (m < 1 || m > 16 || n < 8 || n % 8 != 0 || k < 16 || (k * wbytes) % 16 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 1) || (reinterpret_cast<uintptr_t>(out) & 1)) {
    return false;
  }
  return geometry_for(m, n, k, wbytes, xbytes, has_residual).stages >= 3;
}

}  // namespace

int skinny_plan(int m, int n, int k, int wbytes, int xbytes, int has_residual, int32_t *out) {
  if (m < 1 || m > 16 || n < 8 || n % 8 != 0 || k < 16 || (k * wbytes) % 16 != 0) return 0;
  const Geometry g = geometry_for(m, n, k, wbytes, xbytes, has_residual != 0);
  if (g.stages < 3) return 0;
  out[0] = g.ctas;
  out[1] = 8 << g.wn_log2;           // channels per unit
  out[2] = wk_of(g.wn_log2);         // K slices per stage
  out[3] = g.ks.k_chunks;
  out[4] = g.ks.chunk_bytes;
  out[5] = g.ks.slice_bytes;
  out[6] = g.ks.k_pad;               // in weight bytes
  out[7] = g.pitch_w;
  out[8] = g.stage_stride;
  out[9] = g.stages;
  out[10] = g.one_copy;
  out[11] = row_pitch(g.ks.k_pad / wbytes, xbytes);
  out[12] = g.x_bytes;
  out[13] = g.ep_bytes;
  out[14] = g.grid;
  out[15] = static_cast<int32_t>(g.x_bytes + kFixedSmem + g.ep_bytes + static_cast<long long>(g.stages) * g.stage_stride);
  return 1;
}

bool skinny_fp8_supported(int m, int n, int k, const void *x, const void *w, const void *out, bool has_residual) {
  return supported(m, n, k, 1, 1, x, w, out, has_residual);
}

bool skinny_upcast_supported(int m, int n, int k, const void *x, const void *w, const void *out, bool has_residual) {
  return supported(m, n, k, 1, 2, x, w, out, has_residual);
}

bool skinny_w16_supported(int m, int n, int k, const void *x, const void *w, const void *out, bool has_residual) {
  return supported(m, n, k, 2, 2, x, w, out, has_residual);
}

cudaError_t skinny_fp8_linear(const void *x, int is_bf16, int m, int n, int k, const uint8_t *w, const float *col_scale,
                              int col_scale_scalar, const void *bias, const void *residual, int act, void *out,
                              uint32_t *status, cudaStream_t stream) {
  SkinnyParams p;
  p.x = static_cast<const uint16_t *>(x);
  p.is_bf16 = is_bf16;
  p.w = w;
  p.col_scale = col_scale;
  p.col_scale_scalar = col_scale_scalar;
  p.bias = bias;
  p.residual = residual;
  p.residual_rows = m;
  p.residual_ld = n;
  p.act = act;
  p.out = static_cast<uint16_t *>(out);
  p.m = m;
  p.n = n;
  p.k = k;
  p.status = status;
  return launch<true, false, false>(p, stream);
}

cudaError_t skinny_upcast_matmul(const void *x, int is_bf16, int m, int n, int k, const uint8_t *w, const float *scale,
                                 const void *bias, const void *residual, int residual_rows, int64_t residual_ld,
                                 void *out, uint32_t *status, cudaStream_t stream) {
  SkinnyParams p;
  p.x = static_cast<const uint16_t *>(x);
  p.is_bf16 = is_bf16;
  p.w = w;
  p.col_scale = scale;
  p.col_scale_scalar = 1;
  p.bias = bias;
  p.residual = residual;
  p.residual_rows = residual_rows > 0 ? residual_rows : m;
  p.residual_ld = residual_ld;
  p.act = 0;
  p.out = static_cast<uint16_t *>(out);
  p.m = m;
  p.n = n;
  p.k = k;
  p.status = status;
  return is_bf16 ? launch<false, true, false>(p, stream) : launch<false, false, false>(p, stream);
}

cudaError_t skinny_w16_matmul(const void *x, int is_bf16, int m, int n, int k, const void *w, const void *bias,
                              const void *residual, int residual_rows, int64_t residual_ld, void *out,
                              uint32_t *status, cudaStream_t stream) {
  SkinnyParams p;
  p.x = static_cast<const uint16_t *>(x);
  p.is_bf16 = is_bf16;
  p.w = static_cast<const uint8_t *>(w);
  p.col_scale = nullptr;
  p.col_scale_scalar = 0;
  p.bias = bias;
  p.residual = residual;
  p.residual_rows = residual_rows > 0 ? residual_rows : m;
  p.residual_ld = residual_ld;
  p.act = 0;
  p.out = static_cast<uint16_t *>(out);
  p.m = m;
  p.n = n;
  p.k = k;
  p.status = status;
  return is_bf16 ? launch<false, true, true>(p, stream) : launch<false, false, true>(p, stream);
}

}  // namespace flsm100
