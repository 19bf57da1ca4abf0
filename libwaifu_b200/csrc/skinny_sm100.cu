// The skinny case of the quantized linear: at most 16 activation rows (decode rows, the M = batch
// adaLN modulation and time-embedding linears, waifu/src/qwen_image/dit.rs:464-475,497-504,565).
// With so few rows the product is bound by streaming the weight from HBM once, so this kernel is
// shaped for bandwidth, not for the tensor pipe:
//
//   * one launch does everything: each CTA quantises the activation rows itself (per-token e4m3,
//     the same arithmetic as quantize_fp8_act) into shared memory, so there is no separate
//     quantiser launch and no scratch;
//   * a CTA owns a block of output channels and all of K; its 8 warps split K, and every thread
//     streams the weight with 16-byte loads that are used exactly once (no shared-memory staging
//     of the weight at all);
//   * the arithmetic is the warp-level mma.sync m16n8k32 e4m3 x e4m3 -> fp32 (exact products, fp32
//     accumulation); the K order inside an instruction is permuted so that a thread's 16
//     contiguous weight bytes feed two instructions directly from registers;
//   * partial sums meet in shared memory and the fused epilogue (row and channel scales, bias,
//     GELU-tanh, residual, one rounding) writes the 16-bit result.
//
// The same kernel has an "upcast" form for the reference-compatible fl_fp8_matmul[_add], whose
// activation is not narrowed (flint/capi.cc:1011-1016): the rows stay 16-bit in shared memory,
// the weight's e4m3 bytes are widened to half (or bfloat16) in registers as the reference's
// kernel does (flint/cuda/gemm_fp8_cutlass.cu:20-29), and the instruction is m16n8k16. This is
// the reference's decode shape (1 x 16384 x 3072, docs/fp8.md:225-244).
#include "skinny_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kKStep = 64;  // K bytes one warp consumes per iteration (two MMAs of 32)

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

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

// Two e4m3 bytes (the low 16 bits of `two`) -> two halves / two bfloat16, exactly.
__device__ __forceinline__ uint32_t widen_e4m3x2(uint32_t two, int to_bf16) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(two)));
  if (!to_bf16) return h2;
  const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h2));
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t *>(&b);
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
  int k_pad;             // k rounded up to kKStep
  int pitch;             // bytes between quantised rows in shared memory: k_pad, plus 64 where that
                         // makes it 64 mod 128 (a quarter warp's 16-byte reads then hit distinct banks)
  int rows_smem;         // activation rows kept in shared memory (= m)
  int x_vec;             // x is 16-byte aligned: 16-byte reads of the activation
};

// NCHUNK output channels per CTA (a multiple of 8). UPCAST: the activation stays 16-bit and the
// weight is widened in registers (the reference-compatible product); otherwise the activation is
// quantised per row to e4m3 first.
template <int NCHUNK, bool UPCAST>
__global__ void __launch_bounds__(kThreads) skinny_fp8_kernel(const SkinnyParams p) {
  constexpr int GROUPS = NCHUNK / 8;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t *xq = smem;                                            // [rows_smem][k_pad] e4m3 codes
  float *row_scale = reinterpret_cast<float *>(xq + p.rows_smem * p.pitch);  // [16]
  float *red = row_scale + 16;                                   // [kWarps][16][NCHUNK]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  griddep_wait();
  griddep_launch_dependents();

  // ---- 1. the activation rows into shared memory (a warp per row): quantised per token to e4m3,
  //         or as they are in the upcast form
  for (int r = warp; r < p.rows_smem; r += kWarps) {
    uint8_t *dst = xq + r * p.pitch;
    const uint16_t *src = p.x + static_cast<long long>(r) * p.k;
    if constexpr (UPCAST) {
      for (int i = lane * 8; i < p.k_pad; i += 32 * 8) {  // 8 elements = 16 bytes
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i < p.k) {
          if (p.x_vec) {
            v = *reinterpret_cast<const uint4 *>(src + i);
          } else {
            uint16_t e[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) e[j] = src[i + j];
            v = make_uint4(e[0] | (uint32_t(e[1]) << 16), e[2] | (uint32_t(e[3]) << 16), e[4] | (uint32_t(e[5]) << 16),
                           e[6] | (uint32_t(e[7]) << 16));
          }
        }
        *reinterpret_cast<uint4 *>(dst + 2 * i) = v;
      }
      if (lane == 0) row_scale[r] = 1.0f;
      continue;
    }
    float amax = 0.0f;
    if (p.x_vec) {
      for (int i = lane * 8; i < p.k; i += 32 * 8) {  // k is a multiple of 16
        const uint4 v = *reinterpret_cast<const uint4 *>(src + i);
        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          amax = fmaxf(amax, fabsf(widen16(static_cast<uint16_t>(w4[j] & 0xffff), p.is_bf16)));
          amax = fmaxf(amax, fabsf(widen16(static_cast<uint16_t>(w4[j] >> 16), p.is_bf16)));
        }
      }
    } else {
      for (int i = lane; i < p.k; i += 32) amax = fmaxf(amax, fabsf(widen16(src[i], p.is_bf16)));
    }
    amax = warp_max(amax);
    const float scale = __fdiv_rn(amax, 448.0f);
    const float inv = __frcp_rn(scale > 0.0f ? scale : 1.0f);
    if (lane == 0) row_scale[r] = scale;
    for (int i = lane * 8; i < p.k_pad; i += 32 * 8) {
      uint32_t lo = 0, hi = 0;
      if (i < p.k) {  // a group of 8 is whole or absent
        uint16_t e[8];
        if (p.x_vec) {
          const uint4 v = *reinterpret_cast<const uint4 *>(src + i);
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            e[2 * j] = static_cast<uint16_t>(w4[j] & 0xffff);
            e[2 * j + 1] = static_cast<uint16_t>(w4[j] >> 16);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = src[i + j];
        }
        uint32_t two[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 pair = make_float2(__fmul_rn(widen16(e[2 * j], p.is_bf16), inv), __fmul_rn(widen16(e[2 * j + 1], p.is_bf16), inv));
          two[j] = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(pair, __NV_SATFINITE, __NV_E4M3)) & 0xffff;
        }
        lo = two[0] | (two[1] << 16);
        hi = two[2] | (two[3] << 16);
      }
      *reinterpret_cast<uint2 *>(dst + i) = make_uint2(lo, hi);
    }
  }
  for (int r = p.rows_smem + threadIdx.x; r < 16; r += kThreads) row_scale[r] = 0.0f;
  __syncthreads();
  const bool row_lo = (threadIdx.x & 31) / 4 < p.rows_smem;      // fragment row g is a real row
  const bool row_hi = (threadIdx.x & 31) / 4 + 8 < p.rows_smem;  // fragment row g + 8 is a real row

  // ---- 2. stream this CTA's weight rows; warps split K
  const int n0 = blockIdx.x * NCHUNK;
  const int steps = p.k_pad / kKStep;
  const int per_warp = (steps + kWarps - 1) / kWarps;
  const int s0 = warp * per_warp;
  const int s1 = min(steps, s0 + per_warp);
  const int g = lane >> 2;  // row of the A fragment / column of the B fragment
  const int q = lane & 3;   // which 16 of the step's 64 K bytes this thread holds
  float acc[GROUPS][4];
#pragma unroll
  for (int j = 0; j < GROUPS; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

  for (int s = s0; s < s1; ++s) {
    const int kbyte = s * kKStep + q * 16;
    // Weight: 16 contiguous bytes of row n0 + 8 j + g for every channel group, all issued before
    // any is used. Read once, so keep it out of L1.
    uint4 wv[GROUPS];
    const bool k_ok = kbyte < p.k;  // k is a multiple of 16: a 16-byte piece is whole or absent
#pragma unroll
    for (int j = 0; j < GROUPS; ++j) {
      const int n = n0 + j * 8 + g;
      if (k_ok && n < p.n) {
        wv[j] = __ldcs(reinterpret_cast<const uint4 *>(p.w + static_cast<long long>(n) * p.k + kbyte));
      } else {
        wv[j] = make_uint4(0, 0, 0, 0);
      }
    }
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    if constexpr (UPCAST) {
      // 16 halves of row g (and g + 8) for this thread's 16 K positions.
      const uint8_t *xr = xq + 2 * kbyte;
      const uint4 xa0 = row_lo ? *reinterpret_cast<const uint4 *>(xr + g * p.pitch) : zero4;
      const uint4 xa1 = row_lo ? *reinterpret_cast<const uint4 *>(xr + g * p.pitch + 16) : zero4;
      const uint4 xb0 = row_hi ? *reinterpret_cast<const uint4 *>(xr + (g + 8) * p.pitch) : zero4;
      const uint4 xb1 = row_hi ? *reinterpret_cast<const uint4 *>(xr + (g + 8) * p.pitch + 16) : zero4;
      const uint32_t al[8] = {xa0.x, xa0.y, xa0.z, xa0.w, xa1.x, xa1.y, xa1.z, xa1.w};
      const uint32_t ah[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
      // Instruction i takes K positions 4i..4i+3 of the thread's 16: the first pair is its "low"
      // half and the second its "high" half, for A and for B alike.
#pragma unroll
      for (int j = 0; j < GROUPS; ++j) {
        const uint32_t wb[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t b0 = widen_e4m3x2(wb[i] & 0xffff, p.is_bf16);
          const uint32_t b1 = widen_e4m3x2(wb[i] >> 16, p.is_bf16);
          if (p.is_bf16) mma_bf16(acc[j], al[2 * i], ah[2 * i], al[2 * i + 1], ah[2 * i + 1], b0, b1);
          else mma_f16(acc[j], al[2 * i], ah[2 * i], al[2 * i + 1], ah[2 * i + 1], b0, b1);
        }
      }
    } else {
      const uint4 xa = row_lo ? *reinterpret_cast<const uint4 *>(xq + g * p.pitch + kbyte) : zero4;
      const uint4 xb = row_hi ? *reinterpret_cast<const uint4 *>(xq + (g + 8) * p.pitch + kbyte) : zero4;
      // Logical k of an instruction <-> physical byte: registers (x, y) of the 16 bytes are the
      // "low" and "high" halves of the first instruction, (z, w) of the second. The same
      // permutation is applied to A and B, so every product pairs the same physical k.
#pragma unroll
      for (int j = 0; j < GROUPS; ++j) {
        mma_e4m3(acc[j], xa.x, xb.x, xa.y, xb.y, wv[j].x, wv[j].y);
        mma_e4m3(acc[j], xa.z, xb.z, xa.w, xb.w, wv[j].z, wv[j].w);
      }
    }
  }

  // ---- 3. partial sums of the warps meet in shared memory
  float *mine = red + warp * 16 * NCHUNK;
#pragma unroll
  for (int j = 0; j < GROUPS; ++j) {
    const int c = j * 8 + q * 2;
    mine[g * NCHUNK + c] = acc[j][0];
    mine[g * NCHUNK + c + 1] = acc[j][1];
    mine[(g + 8) * NCHUNK + c] = acc[j][2];
    mine[(g + 8) * NCHUNK + c + 1] = acc[j][3];
  }
  __syncthreads();

  // ---- 4. fused epilogue
  for (int idx = threadIdx.x; idx < p.m * NCHUNK; idx += kThreads) {
    const int r = idx / NCHUNK;
    const int c = idx - r * NCHUNK;
    const int n = n0 + c;
    if (n >= p.n) continue;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) v += red[w * 16 * NCHUNK + r * NCHUNK + c];
    const float cs = p.col_scale ? (p.col_scale_scalar ? __ldg(p.col_scale) : __ldg(p.col_scale + n)) : 1.0f;
    v = v * (row_scale[r] * cs);
    const long long o = static_cast<long long>(r) * p.n + n;
    if (p.bias) {
      v += p.is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.bias)[n])
                     : __half2float(reinterpret_cast<const __half *>(p.bias)[n]);
    }
    if (p.act == 1) v = gelu_tanh(v);
    if (p.residual) {
      const long long ro = static_cast<long long>(r % p.residual_rows) * p.residual_ld + n;
      v += p.is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.residual)[ro])
                     : __half2float(reinterpret_cast<const __half *>(p.residual)[ro]);
    }
    p.out[o] = p.is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
  }
}

template <int NCHUNK, bool UPCAST>
cudaError_t launch(const SkinnyParams &p, size_t smem, cudaStream_t stream) {
  auto kernel = skinny_fp8_kernel<NCHUNK, UPCAST>;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((p.n + NCHUNK - 1) / NCHUNK), 1, 1);
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

// Bytes between activation rows in shared memory: the row itself, plus 64 where that makes the
// pitch 64 mod 128 so that a quarter warp's 16-byte reads of two rows hit distinct banks.
int row_pitch(int k_pad, bool upcast) {
  const int row = upcast ? 2 * k_pad : k_pad;
  return row + (row % 128 == 0 ? 64 : 0);
}

size_t smem_bytes(int m, int k, bool upcast, int nchunk) {
  const int k_pad = (k + kKStep - 1) / kKStep * kKStep;
  return static_cast<size_t>(m) * row_pitch(k_pad, upcast) + 64 + static_cast<size_t>(kWarps) * 16 * nchunk * 4;
}

template <bool UPCAST>
cudaError_t dispatch(SkinnyParams &p, cudaStream_t stream) {
  p.k_pad = (p.k + kKStep - 1) / kKStep * kKStep;
  p.pitch = row_pitch(p.k_pad, UPCAST);
  p.rows_smem = p.m;
  p.x_vec = (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 ? 1 : 0;
  // Enough CTAs to keep every SM streaming: 64 channels per CTA while that still gives two CTAs
  // per SM, fewer channels per CTA for smaller weights.
  const int sms = 148;
  if (p.n / 64 >= 2 * sms) return launch<64, UPCAST>(p, smem_bytes(p.m, p.k, UPCAST, 64), stream);
  if (p.n / 32 >= sms) return launch<32, UPCAST>(p, smem_bytes(p.m, p.k, UPCAST, 32), stream);
  if (p.n / 16 >= sms) return launch<16, UPCAST>(p, smem_bytes(p.m, p.k, UPCAST, 16), stream);
  return launch<8, UPCAST>(p, smem_bytes(p.m, p.k, UPCAST, 8), stream);
}

bool supported(int m, int n, int k, const void *x, const void *w, const void *out, bool upcast) {
  if (m < 1 || m > 16 || n % 8 != 0 || k % 16 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 1) || (reinterpret_cast<uintptr_t>(out) & 1)) {
    return false;
  }
  return smem_bytes(m, k, upcast, 64) <= 200 * 1024;
}

}  // namespace

bool skinny_fp8_supported(int m, int n, int k, const void *x, const void *w, const void *out) {
  return supported(m, n, k, x, w, out, false);
}

bool skinny_upcast_supported(int m, int n, int k, const void *x, const void *w, const void *out) {
  return supported(m, n, k, x, w, out, true);
}

cudaError_t skinny_fp8_linear(const void *x, int is_bf16, int m, int n, int k, const uint8_t *w, const float *col_scale,
                              int col_scale_scalar, const void *bias, const void *residual, int act, void *out,
                              cudaStream_t stream) {
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
  return dispatch<false>(p, stream);
}

cudaError_t skinny_upcast_matmul(const void *x, int is_bf16, int m, int n, int k, const uint8_t *w, const float *scale,
                                 const void *bias, const void *residual, int residual_rows, int64_t residual_ld,
                                 void *out, cudaStream_t stream) {
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
  return dispatch<true>(p, stream);
}

}  // namespace flsm100
