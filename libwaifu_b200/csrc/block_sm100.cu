// Steps of a transformer block between two of its projections (see block_sm100.cuh).
#include "block_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace flsm100 {

namespace {

__device__ __forceinline__ float widen(uint16_t v, int is_bf16) {
  if (is_bf16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  return __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ uint16_t narrow(float v, int is_bf16) {
  return is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

// One CTA row of the grid per row of qkv. A head is spread over LPH = head_dim / 8 lanes, 8
// consecutive elements (four pairs, one 16-byte vector) per lane, so a warp holds 32 / LPH heads at
// a time and takes kUnits such groups: all their vector loads are issued before the first is used,
// which is what keeps enough bytes in flight for a kernel with this little work per byte, and no
// index needs a division. A CTA reads and writes one contiguous run of the row (the v third aside).
constexpr int kUnits = 2;
constexpr int kMaxWarps = 16;

// Two float32 values in one 64-bit register and instructions that work on both lanes at once, each
// lane rounded as the scalar instruction rounds it: this kernel is bound by instruction issue.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float *lo, float *hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t bf16x2_widen(uint32_t w) {
  return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ uint32_t bf16x2_narrow(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// The kernel below for bfloat16 rows, a pair (one 32-bit word: the even and the odd element of a
// rotation) at a time: the same operations per element in the same order, the head's sum of
// squares kept in two lanes that are added before the shuffles.
template <int LPH>
__global__ void __launch_bounds__(kMaxWarps * 32) qk_norm_rope_bf16_kernel(uint16_t *__restrict__ qkv, int heads, int tokens,
                                                                         const uint16_t *__restrict__ q_weight,
                                                                         const uint16_t *__restrict__ k_weight,
                                                                         const float *__restrict__ cos,
                                                                         const float *__restrict__ sin, float eps) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int HEAD_DIM = LPH * 8;
  constexpr int HPW = 32 / LPH;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPH;
  const int part = lane % LPH;
  const int per_row = 2 * heads;
  const int first = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kUnits * HPW;
  const int64_t row = blockIdx.x;
  const int pos = static_cast<int>(blockIdx.x % static_cast<unsigned>(tokens));

  uint16_t *p[kUnits];
  uint4 raw[kUnits];
#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
    const int slot = first + u * HPW + sub;
    p[u] = nullptr;
    if (slot < per_row) {
      p[u] = qkv + row * (3LL * heads * HEAD_DIM) + static_cast<int64_t>(slot) * HEAD_DIM + part * 8;
      raw[u] = *reinterpret_cast<const uint4 *>(p[u]);
    } else {
      raw[u] = make_uint4(0, 0, 0, 0);
    }
  }
  const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cos + static_cast<int64_t>(pos) * (HEAD_DIM / 2)) + part);
  const float4 s4 = __ldg(reinterpret_cast<const float4 *>(sin + static_cast<int64_t>(pos) * (HEAD_DIM / 2)) + part);
  const uint64_t cc[4] = {f2_pack(c4.x, c4.x), f2_pack(c4.y, c4.y), f2_pack(c4.z, c4.z), f2_pack(c4.w, c4.w)};
  const uint64_t sn[4] = {f2_pack(s4.x, s4.x), f2_pack(s4.y, s4.y), f2_pack(s4.z, s4.z), f2_pack(s4.w, s4.w)};

#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
    const int slot = first + u * HPW + sub;
    const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
    uint64_t f[4];
    uint64_t ss2 = f2_pack(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[i] = bf16x2_widen(w4[i]);
      ss2 = f2_fma(f[i], f[i], ss2);
    }
    float ss, ss_hi;
    f2_unpack(ss2, &ss, &ss_hi);
    ss += ss_hi;
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!p[u]) continue;
    const uint16_t *weight = slot < heads ? q_weight : k_weight;
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(HEAD_DIM)), eps)));
    const uint64_t inv2 = f2_pack(inv, inv);
    if (weight) {
      const uint4 wq = __ldg(reinterpret_cast<const uint4 *>(weight) + part);
      const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] = f2_mul(f[i], bf16x2_widen(ww[i]));
    }
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a, b;
      f2_unpack(f2_mul(f[j], inv2), &a, &b);
      const uint64_t n = bf16x2_widen(bf16x2_narrow(a, b));  // the norm's 16-bit output: (even, odd)
      float ec, oc, es, os;
      f2_unpack(f2_mul(n, cc[j]), &ec, &oc);
      f2_unpack(f2_mul(n, sn[j]), &es, &os);
      out[j] = bf16x2_narrow(__fsub_rn(ec, os), __fadd_rn(es, oc));
    }
    *reinterpret_cast<uint4 *>(p[u]) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

template <int LPH>
__global__ void __launch_bounds__(kMaxWarps * 32) qk_norm_rope_kernel(uint16_t *__restrict__ qkv, int is_bf16,
                                                                    int heads, int tokens,
                                                                    const uint16_t *__restrict__ q_weight,
                                                                    const uint16_t *__restrict__ k_weight,
                                                                    const float *__restrict__ cos, const float *__restrict__ sin,
                                                                    float eps) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int HEAD_DIM = LPH * 8;
  constexpr int HPW = 32 / LPH;  // heads per warp and unit
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPH;      // which of the warp's heads
  const int part = lane % LPH;     // which 8 elements of the head
  const int per_row = 2 * heads;   // q heads then k heads: the first two thirds of the row
  const int first = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kUnits * HPW;
  const int64_t row = blockIdx.x;
  const int pos = static_cast<int>(blockIdx.x % static_cast<unsigned>(tokens));

  uint16_t *p[kUnits];
  uint4 raw[kUnits];
#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
    const int slot = first + u * HPW + sub;
    p[u] = nullptr;
    if (slot < per_row) {
      p[u] = qkv + row * (3LL * heads * HEAD_DIM) + static_cast<int64_t>(slot) * HEAD_DIM + part * 8;
      raw[u] = *reinterpret_cast<const uint4 *>(p[u]);
    } else {
      raw[u] = make_uint4(0, 0, 0, 0);
    }
  }
  // this lane's four pairs of the tables (the same for every head of the row)
  const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cos + static_cast<int64_t>(pos) * (HEAD_DIM / 2)) + part);
  const float4 s4 = __ldg(reinterpret_cast<const float4 *>(sin + static_cast<int64_t>(pos) * (HEAD_DIM / 2)) + part);
  const float cj[4] = {c4.x, c4.y, c4.z, c4.w};
  const float sj[4] = {s4.x, s4.y, s4.z, s4.w};

#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
    const int slot = first + u * HPW + sub;
    const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
    float f[8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = widen(static_cast<uint16_t>(w4[i] & 0xffff), is_bf16);
      f[2 * i + 1] = widen(static_cast<uint16_t>(w4[i] >> 16), is_bf16);
      ss += f[2 * i] * f[2 * i] + f[2 * i + 1] * f[2 * i + 1];
    }
    // every lane takes part in the shuffles, whether its head exists or not
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!p[u]) continue;
    const uint16_t *weight = slot < heads ? q_weight : k_weight;
    // One IEEE reciprocal per head, then a multiplication per element (a division per element
    // would make this kernel ALU-bound).
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(HEAD_DIM)), eps)));
    if (weight) {
      const uint4 wq = __ldg(reinterpret_cast<const uint4 *>(weight) + part);
      const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[2 * i] = __fmul_rn(f[2 * i], widen(static_cast<uint16_t>(ww[i] & 0xffff), is_bf16));
        f[2 * i + 1] = __fmul_rn(f[2 * i + 1], widen(static_cast<uint16_t>(ww[i] >> 16), is_bf16));
      }
    }
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float even = widen(narrow(__fmul_rn(f[2 * j], inv), is_bf16), is_bf16);  // the norm's 16-bit output
      const float odd = widen(narrow(__fmul_rn(f[2 * j + 1], inv), is_bf16), is_bf16);
      const uint16_t left = narrow(__fsub_rn(__fmul_rn(even, cj[j]), __fmul_rn(odd, sj[j])), is_bf16);
      const uint16_t right = narrow(__fadd_rn(__fmul_rn(even, sj[j]), __fmul_rn(odd, cj[j])), is_bf16);
      out[j] = left | (static_cast<uint32_t>(right) << 16);
    }
    *reinterpret_cast<uint4 *>(p[u]) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

template <int LPH>
cudaError_t launch(void *qkv, int is_bf16, int64_t rows, int heads, int tokens, const void *qw, const void *kw,
                   const float *cos, const float *sin, float eps, cudaStream_t stream) {
  const int per_row = 2 * heads;
  const int per_warp = kUnits * (32 / LPH);
  int warps = (per_row + per_warp - 1) / per_warp;
  if (warps > kMaxWarps) warps = kMaxWarps;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows), static_cast<unsigned>((per_row + warps * per_warp - 1) / (warps * per_warp)), 1);
  cfg.blockDim = dim3(static_cast<unsigned>(warps * 32), 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (is_bf16) {
    return cudaLaunchKernelEx(&cfg, qk_norm_rope_bf16_kernel<LPH>, static_cast<uint16_t *>(qkv), heads, tokens,
                              static_cast<const uint16_t *>(qw), static_cast<const uint16_t *>(kw), cos, sin, eps);
  }
  return cudaLaunchKernelEx(&cfg, qk_norm_rope_kernel<LPH>, static_cast<uint16_t *>(qkv), is_bf16, heads, tokens,
                            static_cast<const uint16_t *>(qw), static_cast<const uint16_t *>(kw), cos, sin, eps);
}

}  // namespace

cudaError_t qk_norm_rope(void *qkv, int is_bf16, int64_t rows, int heads, int head_dim, int tokens,
                         const void *q_weight, const void *k_weight, const float *cos, const float *sin, float eps,
                         cudaStream_t stream) {
  switch (head_dim) {
    case 64: return launch<8>(qkv, is_bf16, rows, heads, tokens, q_weight, k_weight, cos, sin, eps, stream);
    case 128: return launch<16>(qkv, is_bf16, rows, heads, tokens, q_weight, k_weight, cos, sin, eps, stream);
    case 256: return launch<32>(qkv, is_bf16, rows, heads, tokens, q_weight, k_weight, cos, sin, eps, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace flsm100
