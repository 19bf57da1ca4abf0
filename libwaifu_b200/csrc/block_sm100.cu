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

// One CTA row of the grid per row of qkv; a warp takes kUnits consecutive q or k heads of it,
// EPL = head_dim / 32 consecutive elements (EPL / 2 pairs) per lane and head: all the heads' vector
// loads are issued before the first is used, which is what keeps enough bytes in flight for a
// kernel with this little work per byte, and no index needs a division. A CTA reads and writes
// one contiguous run of the row (the v third aside).
constexpr int kUnits = 4;
constexpr int kMaxWarps = 16;

template <int EPL>
__global__ void __launch_bounds__(kMaxWarps * 32) qk_norm_rope_kernel(uint16_t *__restrict__ qkv, int is_bf16,
                                                                    int heads, int tokens, const uint16_t *__restrict__ q_weight,
                                                         const uint16_t *__restrict__ k_weight,
                                                         const float *__restrict__ cos, const float *__restrict__ sin,
                                                         float eps) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int HEAD_DIM = EPL * 32;
  constexpr int VEC = EPL == 2 ? 1 : EPL / 4;  // 8-byte vectors per lane and unit (one 4-byte word when EPL == 2)
  const int lane = threadIdx.x & 31;
  const int per_row = 2 * heads;  // q heads then k heads: the first two thirds of the row
  const int first = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kUnits;
  const int64_t row = blockIdx.x;
  const int pos = static_cast<int>(blockIdx.x % static_cast<unsigned>(tokens));

  uint16_t *p[kUnits];
  uint2 raw[kUnits][VEC];
#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
    const int slot = first + u;
    p[u] = nullptr;
    if (slot < per_row) {
      p[u] = qkv + row * (3LL * heads * HEAD_DIM) + static_cast<int64_t>(slot) * HEAD_DIM + lane * EPL;
      if constexpr (EPL == 2) {
        raw[u][0] = make_uint2(*reinterpret_cast<const uint32_t *>(p[u]), 0);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) raw[u][i] = reinterpret_cast<const uint2 *>(p[u])[i];
      }
    }
  }

#pragma unroll
  for (int u = 0; u < kUnits; ++u) {
    if (!p[u]) continue;  // warp-uniform
    const uint16_t *weight = first + u < heads ? q_weight : k_weight;
    uint16_t e[EPL];
    if constexpr (EPL == 2) {
      e[0] = static_cast<uint16_t>(raw[u][0].x & 0xffff);
      e[1] = static_cast<uint16_t>(raw[u][0].x >> 16);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        e[4 * i] = static_cast<uint16_t>(raw[u][i].x & 0xffff);
        e[4 * i + 1] = static_cast<uint16_t>(raw[u][i].x >> 16);
        e[4 * i + 2] = static_cast<uint16_t>(raw[u][i].y & 0xffff);
        e[4 * i + 3] = static_cast<uint16_t>(raw[u][i].y >> 16);
      }
    }
    float f[EPL];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      f[i] = widen(e[i], is_bf16);
      ss += f[i] * f[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    // One IEEE reciprocal per head, then a multiplication per element (a division per element
    // would make this kernel ALU-bound).
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(HEAD_DIM)), eps)));
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      float v = f[i];
      if (weight) v = __fmul_rn(v, widen(__ldg(weight + lane * EPL + i), is_bf16));
      f[i] = widen(narrow(__fmul_rn(v, inv), is_bf16), is_bf16);  // the norm's 16-bit output
    }
    const float *c = cos + static_cast<int64_t>(pos) * (HEAD_DIM / 2) + lane * (EPL / 2);
    const float *s = sin + static_cast<int64_t>(pos) * (HEAD_DIM / 2) + lane * (EPL / 2);
#pragma unroll
    for (int j = 0; j < EPL / 2; ++j) {
      const float cj = __ldg(c + j), sj = __ldg(s + j);
      const float even = f[2 * j], odd = f[2 * j + 1];
      e[2 * j] = narrow(__fsub_rn(__fmul_rn(even, cj), __fmul_rn(odd, sj)), is_bf16);
      e[2 * j + 1] = narrow(__fadd_rn(__fmul_rn(even, sj), __fmul_rn(odd, cj)), is_bf16);
    }
    if constexpr (EPL == 2) {
      *reinterpret_cast<uint32_t *>(p[u]) = e[0] | (static_cast<uint32_t>(e[1]) << 16);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        reinterpret_cast<uint2 *>(p[u])[i] = make_uint2(e[4 * i] | (static_cast<uint32_t>(e[4 * i + 1]) << 16),
                                                        e[4 * i + 2] | (static_cast<uint32_t>(e[4 * i + 3]) << 16));
      }
    }
  }
}

template <int EPL>
cudaError_t launch(void *qkv, int is_bf16, int64_t rows, int heads, int tokens, const void *qw, const void *kw,
                   const float *cos, const float *sin, float eps, cudaStream_t stream) {
  const int per_row = 2 * heads;
  int warps = (per_row + kUnits - 1) / kUnits;
  if (warps > kMaxWarps) warps = kMaxWarps;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows), static_cast<unsigned>((per_row + warps * kUnits - 1) / (warps * kUnits)), 1);
  cfg.blockDim = dim3(static_cast<unsigned>(warps * 32), 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, qk_norm_rope_kernel<EPL>, static_cast<uint16_t *>(qkv), is_bf16, heads, tokens,
                            static_cast<const uint16_t *>(qw), static_cast<const uint16_t *>(kw), cos, sin, eps);
}

}  // namespace

cudaError_t qk_norm_rope(void *qkv, int is_bf16, int64_t rows, int heads, int head_dim, int tokens,
                         const void *q_weight, const void *k_weight, const float *cos, const float *sin, float eps,
                         cudaStream_t stream) {
  switch (head_dim) {
    case 64: return launch<2>(qkv, is_bf16, rows, heads, tokens, q_weight, k_weight, cos, sin, eps, stream);
    case 128: return launch<4>(qkv, is_bf16, rows, heads, tokens, q_weight, k_weight, cos, sin, eps, stream);
    case 256: return launch<8>(qkv, is_bf16, rows, heads, tokens, q_weight, k_weight, cos, sin, eps, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace flsm100
