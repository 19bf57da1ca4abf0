// Helper kernels of the quantized-linear path. All of them are HBM-bound streaming kernels:
// 16-byte vector accesses, one pass where the row fits in registers' reach of L1, grids sized by
// rows. Divisions and reciprocals are IEEE (this file is compiled without fast-math) because the
// codes must be bit-identical to the CPU oracle's; the dynamic quantisers take one reciprocal per
// row or block and multiply by it, which is what keeps them bandwidth-bound.
#include "quant_sm100.cuh"

#include "ptx_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <atomic>

namespace flsm100 {

namespace {

std::atomic<int64_t> g_helper_launches{0};

__device__ __forceinline__ float widen(uint16_t v, int is_bf16) {
  if (is_bf16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  return __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float block_max(float v, float *red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? red[lane] : 0.0f;
  r = warp_max(r);
  __syncthreads();
  return r;
}

__device__ __forceinline__ uint8_t e4m3_of(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float e4m3_value(uint8_t code) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(code), __NV_E4M3);
  return __half2float(__half(h));
}

// Eight 16-bit values times `inv`, as eight e4m3 codes in memory order.
__device__ __forceinline__ uint2 e4m3x8_of(uint4 q, int is_bf16, float inv) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint32_t out[2] = {0, 0};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 pair = make_float2(__fmul_rn(widen(static_cast<uint16_t>(w[j] & 0xffff), is_bf16), inv),
                                    __fmul_rn(widen(static_cast<uint16_t>(w[j] >> 16), is_bf16), inv));
    // x in the low byte, y in the high byte
    const uint32_t two = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(pair, __NV_SATFINITE, __NV_E4M3));
    out[j >> 1] |= (two & 0xffff) << ((j & 1) * 16);
  }
  return make_uint2(out[0], out[1]);
}

// ---- per-row e4m3 ----------------------------------------------------------------------------

// One CTA per row. Pass 1 finds amax, pass 2 re-reads the row (an L1/L2 hit: a row is a few KB)
// and writes the codes. VEC: 16-byte accesses, possible when the bases are 16-byte aligned.
template <bool VEC>
__global__ void __launch_bounds__(128) quantize_fp8_act_kernel(const uint16_t *__restrict__ x, int is_bf16, int k,
                                                             uint8_t *__restrict__ codes,
                                                             float *__restrict__ scales) {
  griddep_wait();
  __shared__ float red[4];
  const int64_t row = blockIdx.x;
  const uint16_t *xr = x + row * k;
  uint8_t *cr = codes + row * k;
  float amax = 0.0f;
  if (VEC) {
    const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
    for (int i = threadIdx.x; i < k / 8; i += blockDim.x) {
      uint4 q = xv[i];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = fmaxf(amax, fabsf(widen(static_cast<uint16_t>(w[j] & 0xffff), is_bf16)));
        amax = fmaxf(amax, fabsf(widen(static_cast<uint16_t>(w[j] >> 16), is_bf16)));
      }
    }
  } else {
    for (int i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(widen(xr[i], is_bf16)));
  }
  amax = block_max(amax, red);
  const float scale = __fdiv_rn(amax, 448.0f);
  const float inv = __frcp_rn(scale > 0.0f ? scale : 1.0f);
  if (threadIdx.x == 0) scales[row] = scale;
  griddep_launch_dependents();
  if (VEC) {
    const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
    uint2 *cv = reinterpret_cast<uint2 *>(cr);
    for (int i = threadIdx.x; i < k / 8; i += blockDim.x) cv[i] = e4m3x8_of(xv[i], is_bf16, inv);
  } else {
    for (int i = threadIdx.x; i < k; i += blockDim.x) cr[i] = e4m3_of(__fmul_rn(widen(xr[i], is_bf16), inv));
  }
}

// The same for rows short enough to stay in registers between the two passes (k <= 2048 * VPT):
// one global read of the row, 256 threads, VPT 16-byte vectors per thread.
template <int VPT>
__global__ void __launch_bounds__(256) quantize_fp8_act_reg_kernel(const uint16_t *__restrict__ x, int is_bf16, int k,
                                                                 uint8_t *__restrict__ codes,
                                                                 float *__restrict__ scales) {
  griddep_wait();
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x + row * k);
  uint2 *cv = reinterpret_cast<uint2 *>(codes + row * k);
  const int nvec = k / 8;
  uint4 q[VPT];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    q[i] = (v < nvec) ? xv[v] : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      amax = fmaxf(amax, fabsf(widen(static_cast<uint16_t>(w[j] & 0xffff), is_bf16)));
      amax = fmaxf(amax, fabsf(widen(static_cast<uint16_t>(w[j] >> 16), is_bf16)));
    }
  }
  amax = block_max(amax, red);
  const float scale = __fdiv_rn(amax, 448.0f);
  const float inv = __frcp_rn(scale > 0.0f ? scale : 1.0f);
  if (threadIdx.x == 0) scales[row] = scale;
  griddep_launch_dependents();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) cv[v] = e4m3x8_of(q[i], is_bf16, inv);
  }
}

// Per-row e4m3 of x (m, k) with the rows' maxima given (taken over a wider row than x: x is one
// rank's column block of a matrix split by output channel, `amax` the maximum over all ranks'
// blocks), written into columns [col0, col0 + k) of up to eight (m, ld) matrices of codes: this
// GPU's own and its peers'. The arithmetic is quantize_fp8_act's, so the gathered codes equal what
// that kernel makes of the whole row. A CTA takes a row; a lane's 16 bytes of codes go out as one
// store per destination, 512 contiguous bytes per warp, which is what NVLink wants.
struct ScatterDests {
  uint8_t *ptr[8];
  int count;
};

__global__ void __launch_bounds__(128) quantize_fp8_scatter_kernel(const uint16_t *__restrict__ x, int is_bf16, int k,
                                                                 const float *__restrict__ amax, ScatterDests dests,
                                                                 long long ld, int col0, float *__restrict__ scales) {
  griddep_wait();
  const long long row = blockIdx.x;
  const float scale = __fdiv_rn(amax[row], 448.0f);
  const float inv = __frcp_rn(scale > 0.0f ? scale : 1.0f);
  if (threadIdx.x == 0 && scales) scales[row] = scale;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x + row * k);
  for (int v = threadIdx.x; v < k / 16; v += blockDim.x) {
    const uint2 lo = e4m3x8_of(xv[2 * v], is_bf16, inv);
    const uint2 hi = e4m3x8_of(xv[2 * v + 1], is_bf16, inv);
    const uint4 codes = make_uint4(lo.x, lo.y, hi.x, hi.y);
    const long long off = row * ld + col0 + static_cast<long long>(v) * 16;
#pragma unroll 1
    for (int d = 0; d < dests.count; ++d) *reinterpret_cast<uint4 *>(dests.ptr[d] + off) = codes;
  }
}

// The largest magnitude of each row of a 16-bit matrix whose rows lie `pitch` elements apart.
__global__ void __launch_bounds__(128) row_amax_kernel(const uint16_t *__restrict__ x, int is_bf16, int k, long long pitch,
                                                     float *__restrict__ amax) {
  __shared__ float red[4];
  const uint16_t *xr = x + blockIdx.x * pitch;
  uint32_t top = 0;  // magnitudes of one 16-bit format order like their bit patterns
  if ((reinterpret_cast<uintptr_t>(xr) & 15) == 0 && k % 8 == 0) {
    const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
    for (int v = threadIdx.x; v < k / 8; v += blockDim.x) {
      const uint4 q = xv[v];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) top = max(top, max(w[j] & 0x7fffu, (w[j] >> 16) & 0x7fffu));
    }
  } else {
    for (int i = threadIdx.x; i < k; i += blockDim.x) top = max(top, static_cast<uint32_t>(xr[i]) & 0x7fffu);
  }
  const float mine = widen(static_cast<uint16_t>(top), is_bf16);
  const float all = block_max(mine, red);
  if (threadIdx.x == 0) amax[blockIdx.x] = all;
}

// ---- layer norm -> modulate -> per-row e4m3, one pass ----------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Two sums at once: one pair of barriers for both.
__device__ __forceinline__ float2 block_sum2(float a, float b, float2 *red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (lane == 0) red[warp] = make_float2(a, b);
  __syncthreads();
  float2 r = (lane < nwarps) ? red[lane] : make_float2(0.0f, 0.0f);
  r.x = warp_sum(r.x);
  r.y = warp_sum(r.y);
  __syncthreads();
  return r;
}

// The reference's statistics (flint/cpu/normalizations.cc:126-137): mean = sum / k,
// variance = sumsq / k - mean^2, 1 / sqrt(variance + eps), with eps alone where rounding left the
// variance at or below zero.
__device__ __forceinline__ float2 mean_rstd(float2 sums, int k, float eps) {
  const float mean = __fdiv_rn(sums.x, static_cast<float>(k));
  const float var = __fsub_rn(__fdiv_rn(sums.y, static_cast<float>(k)), __fmul_rn(mean, mean));
  return make_float2(mean, __frcp_rn(__fsqrt_rn(var > 0.0f ? __fadd_rn(var, eps) : eps)));
}

__device__ __forceinline__ uint16_t narrow(float v, int is_bf16) {
  return is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

// One element of the modulated row: ((v - mean) rstd) (x) (1 + s) (+) t, every operation rounded
// on its own in the order the reference's graph applies them (normed * scale + normed, then the
// cast to the narrow type; waifu/src/qwen_image/dit.rs:179-184), as a 16-bit value.
__device__ __forceinline__ uint16_t modulated(float v, float mean, float rstd, const uint16_t *s, const uint16_t *t,
                                              int i, int is_bf16) {
  float y = __fmul_rn(__fsub_rn(v, mean), rstd);
  if (s) y = __fadd_rn(__fmul_rn(y, widen(__ldg(s + i), is_bf16)), y);
  if (t) y = __fadd_rn(y, widen(__ldg(t + i), is_bf16));
  return narrow(y, is_bf16);
}

// One CTA of THREADS threads per row, the row in registers throughout (k <= 8 THREADS VPT): one read of x,
// one block reduction for the two sums of the statistics, one for amax of the modulated 16-bit
// row, one write of the codes. Short rows take 128 threads: more rows in flight per SM, which is
// what a kernel made of a load, two barriers and a store needs to fill the memory pipe.
template <int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS) ln_modulate_quantize_reg_kernel(const uint16_t *__restrict__ x, int is_bf16, int k,
                                                                     const uint16_t *__restrict__ scale,
                                                                     const uint16_t *__restrict__ shift,
                                                                     int rows_per_group, int64_t scale_pitch,
                                                                     int64_t shift_pitch, float eps,
                                                                     uint8_t *__restrict__ codes,
                                                                     float *__restrict__ row_scales) {
  griddep_wait();
  __shared__ float red[8];
  __shared__ float2 red2[8];
  const int64_t row = blockIdx.x;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x + row * k);
  uint2 *cv = reinterpret_cast<uint2 *>(codes + row * k);
  const int64_t group = row / rows_per_group;
  const uint16_t *s = scale ? scale + group * scale_pitch : nullptr;  // a group's row may sit in a wider tensor
  const uint16_t *t = shift ? shift + group * shift_pitch : nullptr;
  const int nvec = k / 8;
  uint4 q[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    q[i] = (v < nvec) ? xv[v] : make_uint4(0, 0, 0, 0);
  }
  float sum = 0.0f, sq = 0.0f;  // the zero padding of the last vectors adds nothing to either
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = widen(static_cast<uint16_t>(w[j] & 0xffff), is_bf16);
      const float hi = widen(static_cast<uint16_t>(w[j] >> 16), is_bf16);
      sum += lo + hi;
      sq += lo * lo + hi * hi;
    }
  }
  const float2 stats = mean_rstd(block_sum2(sum, sq, red2), k, eps);
  const float mean = stats.x, rstd = stats.y;
  // The modulated row replaces x in the registers, already narrowed to the 16-bit type. scale and
  // shift come as the same 16-byte vectors as x (their rows are 16-byte aligned: the host checks).
  float amax = 0.0f;
  const uint4 *sv = reinterpret_cast<const uint4 *>(s);
  const uint4 *tv = reinterpret_cast<const uint4 *>(t);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
      const uint4 s4 = s ? __ldg(sv + v) : make_uint4(0, 0, 0, 0);
      const uint4 t4 = t ? __ldg(tv + v) : make_uint4(0, 0, 0, 0);
      const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
      const uint32_t tw[4] = {t4.x, t4.y, t4.z, t4.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint16_t h[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int sh = half * 16;
          float y = __fmul_rn(__fsub_rn(widen(static_cast<uint16_t>(w[j] >> sh), is_bf16), mean), rstd);
          if (s) y = __fadd_rn(__fmul_rn(y, widen(static_cast<uint16_t>(sw[j] >> sh), is_bf16)), y);
          if (t) y = __fadd_rn(y, widen(static_cast<uint16_t>(tw[j] >> sh), is_bf16));
          h[half] = narrow(y, is_bf16);
          amax = fmaxf(amax, fabsf(widen(h[half], is_bf16)));
        }
        o[j] = h[0] | (static_cast<uint32_t>(h[1]) << 16);
      }
      q[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  amax = block_max(amax, red);
  const float qscale = __fdiv_rn(amax, 448.0f);
  const float inv = __frcp_rn(qscale > 0.0f ? qscale : 1.0f);
  if (threadIdx.x == 0) row_scales[row] = qscale;
  griddep_launch_dependents();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) cv[v] = e4m3x8_of(q[i], is_bf16, inv);
  }
}

// Two float32 values in one 64-bit register and the instructions that work on both lanes at once
// (each lane rounded to nearest even exactly as the scalar instruction rounds it): the row kernels
// are bound by instruction issue, not by memory, and these halve the arithmetic's instructions.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float *lo, float *hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
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
// The two bfloat16 of a 32-bit word, widened: the low one in the low lane.
__device__ __forceinline__ uint64_t bf16x2_widen(uint32_t w) {
  return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// ln_modulate_quantize_reg_kernel for bfloat16 rows with the arithmetic two elements at a time:
// the same operations in the same order per element (v - mean is v + (-mean) bit for bit), the
// statistics summed in two lanes that are added at the end, the row's largest magnitude kept as
// a bfloat16 pair.
template <int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS) ln_modulate_quantize_bf16_kernel(const uint16_t *__restrict__ x, int k,
                                                                      const uint16_t *__restrict__ scale,
                                                                      const uint16_t *__restrict__ shift,
                                                                      int rows_per_group, int64_t scale_pitch,
                                                                      int64_t shift_pitch, float eps,
                                                                      uint8_t *__restrict__ codes,
                                                                      float *__restrict__ row_scales) {
  griddep_wait();
  __shared__ float red[8];
  __shared__ float2 red2[8];
  const int64_t row = blockIdx.x;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x + row * k);
  uint2 *cv = reinterpret_cast<uint2 *>(codes + row * k);
  const int64_t group = row / rows_per_group;
  const uint16_t *s = scale ? scale + group * scale_pitch : nullptr;
  const uint16_t *t = shift ? shift + group * shift_pitch : nullptr;
  const int nvec = k / 8;
  uint4 q[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    q[i] = (v < nvec) ? xv[v] : make_uint4(0, 0, 0, 0);
  }
  uint64_t sum2 = f2_pack(0.0f, 0.0f), sq2 = sum2;  // the zero padding of the last vectors adds nothing to either
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint64_t p = bf16x2_widen(w[j]);
      sum2 = f2_add(sum2, p);
      sq2 = f2_fma(p, p, sq2);
    }
  }
  float s0, s1, q0, q1;
  f2_unpack(sum2, &s0, &s1);
  f2_unpack(sq2, &q0, &q1);
  const float2 stats = mean_rstd(block_sum2(s0 + s1, q0 + q1, red2), k, eps);
  const uint64_t neg_mean2 = f2_pack(-stats.x, -stats.x), rstd2 = f2_pack(stats.y, stats.y);
  __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.0f, 0.0f);
  const uint4 *sv = reinterpret_cast<const uint4 *>(s);
  const uint4 *tv = reinterpret_cast<const uint4 *>(t);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
      const uint4 s4 = s ? __ldg(sv + v) : make_uint4(0, 0, 0, 0);
      const uint4 t4 = t ? __ldg(tv + v) : make_uint4(0, 0, 0, 0);
      const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
      const uint32_t tw[4] = {t4.x, t4.y, t4.z, t4.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint64_t y = f2_mul(f2_add(bf16x2_widen(w[j]), neg_mean2), rstd2);
        if (s) y = f2_add(f2_mul(y, bf16x2_widen(sw[j])), y);
        if (t) y = f2_add(y, bf16x2_widen(tw[j]));
        float y0, y1;
        f2_unpack(y, &y0, &y1);
        const __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
        amax2 = __hmax2(amax2, __habs2(h));
        o[j] = *reinterpret_cast<const uint32_t *>(&h);
      }
      q[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  float amax = fmaxf(__low2float(amax2), __high2float(amax2));
  amax = block_max(amax, red);
  const float qscale = __fdiv_rn(amax, 448.0f);
  const float inv = __frcp_rn(qscale > 0.0f ? qscale : 1.0f);
  if (threadIdx.x == 0) row_scales[row] = qscale;
  griddep_launch_dependents();
  const uint64_t inv2 = f2_pack(inv, inv);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
      uint32_t out[2] = {0, 0};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a, b;
        f2_unpack(f2_mul(bf16x2_widen(w[j]), inv2), &a, &b);
        const uint32_t two = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
        out[j >> 1] |= (two & 0xffff) << ((j & 1) * 16);
      }
      cv[v] = make_uint2(out[0], out[1]);
    }
  }
}

// The same arithmetic for rows of any length and any alignment: the row is read three times (an
// L1/L2 hit after the first) and the modulated value is computed twice.
__global__ void __launch_bounds__(256) ln_modulate_quantize_kernel(const uint16_t *__restrict__ x, int is_bf16, int k,
                                                                 const uint16_t *__restrict__ scale,
                                                                 const uint16_t *__restrict__ shift, int rows_per_group,
                                                                 int64_t scale_pitch, int64_t shift_pitch, float eps,
                                                                 uint8_t *__restrict__ codes,
                                                                 float *__restrict__ row_scales) {
  griddep_wait();
  __shared__ float red[8];
  __shared__ float2 red2[8];
  const int64_t row = blockIdx.x;
  const uint16_t *xr = x + row * k;
  const int64_t group = row / rows_per_group;
  const uint16_t *s = scale ? scale + group * scale_pitch : nullptr;  // a group's row may sit in a wider tensor
  const uint16_t *t = shift ? shift + group * shift_pitch : nullptr;
  float sum = 0.0f, sq = 0.0f;
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const float v = widen(xr[i], is_bf16);
    sum += v;
    sq += v * v;
  }
  const float2 stats = mean_rstd(block_sum2(sum, sq, red2), k, eps);
  const float mean = stats.x, rstd = stats.y;
  float amax = 0.0f;
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    amax = fmaxf(amax, fabsf(widen(modulated(widen(xr[i], is_bf16), mean, rstd, s, t, i, is_bf16), is_bf16)));
  }
  amax = block_max(amax, red);
  const float qscale = __fdiv_rn(amax, 448.0f);
  const float inv = __frcp_rn(qscale > 0.0f ? qscale : 1.0f);
  if (threadIdx.x == 0) row_scales[row] = qscale;
  griddep_launch_dependents();
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const float h = widen(modulated(widen(xr[i], is_bf16), mean, rstd, s, t, i, is_bf16), is_bf16);
    codes[row * k + i] = e4m3_of(__fmul_rn(h, inv));
  }
}

// ---- swiglu -> per-row e4m3, one pass -----------------------------------------------------------

// flint's swiglu on one element pair (flint/cpu/glu.cc:36-67): the first half of the row is the
// gate, the second the value; silu(g) * v with silu(g) = g / (1 + exp(-g)), fp32, narrowed to the
// row's 16-bit type as the operator's output is.
__device__ __forceinline__ uint16_t swiglu16(uint16_t gate, uint16_t value, int is_bf16) {
  const float g = widen(gate, is_bf16);
  const float silu = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
  return narrow(__fmul_rn(silu, widen(value, is_bf16)), is_bf16);
}

// One CTA of 256 threads per row of (2 h): VPT vectors of the gate half and VPT of the value half
// per thread (h <= 2048 VPT), the gated row kept in registers as 16-bit values between the amax
// reduction and the quantisation. One read of the input, one write of the codes.
template <int VPT>
__global__ void __launch_bounds__(256) swiglu_quantize_reg_kernel(const uint16_t *__restrict__ x, int is_bf16, int h,
                                                                uint8_t *__restrict__ codes,
                                                                float *__restrict__ row_scales) {
  griddep_wait();
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const uint4 *gv = reinterpret_cast<const uint4 *>(x + row * 2 * h);
  const uint4 *vv = reinterpret_cast<const uint4 *>(x + row * 2 * h + h);
  uint2 *cv = reinterpret_cast<uint2 *>(codes + row * h);
  const int nvec = h / 8;
  uint4 gq[VPT], vq[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    gq[i] = (v < nvec) ? gv[v] : make_uint4(0, 0, 0, 0);
    vq[i] = (v < nvec) ? vv[v] : make_uint4(0, 0, 0, 0);
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t g[4] = {gq[i].x, gq[i].y, gq[i].z, gq[i].w};
    const uint32_t v[4] = {vq[i].x, vq[i].y, vq[i].z, vq[i].w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint16_t lo = swiglu16(static_cast<uint16_t>(g[j] & 0xffff), static_cast<uint16_t>(v[j] & 0xffff), is_bf16);
      const uint16_t hi = swiglu16(static_cast<uint16_t>(g[j] >> 16), static_cast<uint16_t>(v[j] >> 16), is_bf16);
      amax = fmaxf(amax, fmaxf(fabsf(widen(lo, is_bf16)), fabsf(widen(hi, is_bf16))));
      o[j] = lo | (static_cast<uint32_t>(hi) << 16);
    }
    gq[i] = make_uint4(o[0], o[1], o[2], o[3]);  // zero padding gates to zero
  }
  amax = block_max(amax, red);
  const float qscale = __fdiv_rn(amax, 448.0f);
  const float inv = __frcp_rn(qscale > 0.0f ? qscale : 1.0f);
  if (threadIdx.x == 0) row_scales[row] = qscale;
  griddep_launch_dependents();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) cv[v] = e4m3x8_of(gq[i], is_bf16, inv);
  }
}

// Any length and alignment: the gated value is computed twice.
__global__ void __launch_bounds__(256) swiglu_quantize_kernel(const uint16_t *__restrict__ x, int is_bf16, int h,
                                                            uint8_t *__restrict__ codes,
                                                            float *__restrict__ row_scales) {
  griddep_wait();
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const uint16_t *xr = x + row * 2 * h;
  float amax = 0.0f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) amax = fmaxf(amax, fabsf(widen(swiglu16(xr[i], xr[i + h], is_bf16), is_bf16)));
  amax = block_max(amax, red);
  const float qscale = __fdiv_rn(amax, 448.0f);
  const float inv = __frcp_rn(qscale > 0.0f ? qscale : 1.0f);
  if (threadIdx.x == 0) row_scales[row] = qscale;
  griddep_launch_dependents();
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    codes[row * h + i] = e4m3_of(__fmul_rn(widen(swiglu16(xr[i], xr[i + h], is_bf16), is_bf16), inv));
  }
}

__global__ void __launch_bounds__(128) quantize_fp8_rows_f32_kernel(const float *__restrict__ w, int k,
                                                                  uint8_t *__restrict__ codes,
                                                                  float *__restrict__ scales) {
  __shared__ float red[4];
  const int64_t row = blockIdx.x;
  const float *wr = w + row * k;
  float amax = 0.0f;
  for (int i = threadIdx.x; i < k; i += blockDim.x) amax = fmaxf(amax, fabsf(wr[i]));
  amax = block_max(amax, red);
  const float scale = __fdiv_rn(amax, 448.0f);
  const float divisor = scale > 0.0f ? scale : 1.0f;
  if (threadIdx.x == 0) scales[row] = scale;
  for (int i = threadIdx.x; i < k; i += blockDim.x) codes[row * k + i] = e4m3_of(__fdiv_rn(wr[i], divisor));
}

// ---- NVFP4 -----------------------------------------------------------------------------------

__device__ __forceinline__ int64_t sf_tiled_offset(int r, int b, int sf_k_tiles) {
  return (static_cast<int64_t>(r / 128) * sf_k_tiles + b / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4);
}

// 16 values -> 8 code bytes and the block's scale code, exactly as the oracle's nvfp4_block().
__device__ __forceinline__ uint8_t nvfp4_block(const float (&v)[16], float global, uint32_t (&packed)[2]) {
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
  uint8_t sc = global > 0.0f ? e4m3_of(__fdiv_rn(amax, __fmul_rn(6.0f, global))) : 0;
  const float denom = __fmul_rn(e4m3_value(sc), global);
  packed[0] = packed[1] = 0;
  if (!(denom > 0.0f)) return 0;
  const float inv = __frcp_rn(denom);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float2 pair = make_float2(__fmul_rn(v[2 * j], inv), __fmul_rn(v[2 * j + 1], inv));
    uint32_t byte = static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(pair, __NV_E2M1, cudaRoundNearest));
    packed[j >> 2] |= (byte & 0xff) << ((j & 3) * 8);
  }
  return sc;
}

// Block b of row r of a 16-bit activation: 16 values -> 8 code bytes and the block's scale factor
// in the tile layout.
__device__ __forceinline__ void nvfp4_act_block(const uint16_t *__restrict__ x, int is_bf16, int k, int r, int b,
                                                uint8_t *__restrict__ codes, uint8_t *__restrict__ sf_tiled,
                                                int sf_k_tiles, int vec_ok) {
  const uint16_t *src = x + static_cast<int64_t>(r) * k + 16 * b;
  float v[16];
  if (vec_ok) {
    const uint4 *sv = reinterpret_cast<const uint4 *>(src);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint4 q = sv[h];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[h * 8 + 2 * j] = widen(static_cast<uint16_t>(w[j] & 0xffff), is_bf16);
        v[h * 8 + 2 * j + 1] = widen(static_cast<uint16_t>(w[j] >> 16), is_bf16);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = widen(src[j], is_bf16);
  }
  uint32_t packed[2];
  uint8_t sc = nvfp4_block(v, 1.0f, packed);
  uint8_t *dst = codes + (static_cast<int64_t>(r) * k) / 2 + 8 * b;
  if (vec_ok) {
    *reinterpret_cast<uint2 *>(dst) = make_uint2(packed[0], packed[1]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = static_cast<uint8_t>(packed[j >> 2] >> ((j & 3) * 8));
  }
  sf_tiled[sf_tiled_offset(r, b, sf_k_tiles)] = sc;
}

// One thread per 16-element block of a 16-bit activation.
__global__ void __launch_bounds__(256) quantize_nvfp4_act_kernel(const uint16_t *__restrict__ x, int is_bf16, int m,
                                                               int k, uint8_t *__restrict__ codes,
                                                               uint8_t *__restrict__ sf_tiled, int sf_k_tiles,
                                                               int vec_ok) {
  griddep_wait();
  griddep_launch_dependents();
  const int blocks_per_row = k / 16;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(m) * blocks_per_row) return;
  nvfp4_act_block(x, is_bf16, k, static_cast<int>(idx / blocks_per_row), static_cast<int>(idx % blocks_per_row), codes,
                  sf_tiled, sf_k_tiles, vec_ok);
}

// Everything fl_nvfp4_linear does ahead of its GEMM in one launch (two clears, the activation
// quantiser and the re-tiling of the weight's block scales were four, with a launch gap each).
// CTAs [0, a_ctas): one thread per 16-element block of the activation over the whole tiled domain
// (row groups of 128, K tiles of 4 blocks, `sf_k_tiles` per group): a block of the activation is
// quantised, one of the padding gets the scale factor 0. The other CTAs: one thread per 4 block
// scales of the weight (a 32-bit word of the tile layout) over its tiled domain and one spare row
// group, zeros outside the weight. Nothing has to be cleared beforehand.
__global__ void __launch_bounds__(256) nvfp4_prepare_kernel(const uint16_t *__restrict__ x, int is_bf16, int m, int k,
                                                          uint8_t *__restrict__ codes, uint8_t *__restrict__ sfa_tiled,
                                                          int sf_k_tiles, int vec_ok, int a_ctas,
                                                          const uint8_t *__restrict__ wsf_plain, int rows, int w_groups,
                                                          uint8_t *__restrict__ sfb_tiled) {
  griddep_wait();
  griddep_launch_dependents();
  const int kblocks = k / 16;
  if (static_cast<int>(blockIdx.x) < a_ctas) {
    const int kb_pad = sf_k_tiles * 4;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t total = static_cast<int64_t>((m + 127) / 128) * 128 * kb_pad;
    if (idx >= total) return;
    const int r = static_cast<int>(idx / kb_pad), b = static_cast<int>(idx % kb_pad);
    if (r < m && b < kblocks) {
      nvfp4_act_block(x, is_bf16, k, r, b, codes, sfa_tiled, sf_k_tiles, vec_ok);
    } else {
      sfa_tiled[sf_tiled_offset(r, b, sf_k_tiles)] = 0;
    }
    return;
  }
  const int64_t idx = static_cast<int64_t>(static_cast<int>(blockIdx.x) - a_ctas) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(w_groups) * 128 * sf_k_tiles;
  if (idx >= total) return;
  const int r = static_cast<int>(idx / sf_k_tiles), t4 = static_cast<int>(idx % sf_k_tiles) * 4;
  uint32_t word = 0;
  if (r < rows) {
    const uint8_t *src = wsf_plain + static_cast<int64_t>(r) * kblocks + t4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (t4 + j < kblocks) word |= static_cast<uint32_t>(src[j]) << (8 * j);
    }
  }
  *reinterpret_cast<uint32_t *>(sfb_tiled + sf_tiled_offset(r, t4, sf_k_tiles)) = word;
}

__global__ void __launch_bounds__(256) amax_f32_kernel(const float *__restrict__ w, int64_t numel, uint32_t *amax_word) {
  __shared__ float red[8];
  float amax = 0.0f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    amax = fmaxf(amax, fabsf(w[i]));
  }
  amax = block_max(amax, red);
  // Non-negative floats order like their bit patterns.
  if (threadIdx.x == 0) atomicMax(amax_word, __float_as_uint(amax));
}

__global__ void nvfp4_global_scale_kernel(const uint32_t *amax_word, float *global_scale) {
  *global_scale = __fdiv_rn(__uint_as_float(*amax_word), 448.0f * 6.0f);
}

__global__ void __launch_bounds__(256) quantize_nvfp4_weight_kernel(const float *__restrict__ w, int rows, int k,
                                                                  const float *__restrict__ global_scale,
                                                                  uint8_t *__restrict__ codes,
                                                                  uint8_t *__restrict__ sf_plain) {
  const int blocks_per_row = k / 16;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(rows) * blocks_per_row) return;
  const float *src = w + idx * 16;
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = src[j];
  uint32_t packed[2];
  uint8_t sc = nvfp4_block(v, *global_scale, packed);
  uint8_t *dst = codes + idx * 8;
#pragma unroll
  for (int j = 0; j < 8; ++j) dst[j] = static_cast<uint8_t>(packed[j >> 2] >> ((j & 3) * 8));
  sf_plain[idx] = sc;
}

__global__ void __launch_bounds__(256) pack_sf_kernel(const uint8_t *__restrict__ sf_plain, int rows, int kblocks,
                                                    uint8_t *__restrict__ sf_tiled, int sf_k_tiles) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(rows) * kblocks) return;
  const int r = static_cast<int>(idx / kblocks);
  const int b = static_cast<int>(idx % kblocks);
  sf_tiled[sf_tiled_offset(r, b, sf_k_tiles)] = sf_plain[idx];
}

// ---- widening and gathers --------------------------------------------------------------------

__global__ void __launch_bounds__(256) widen_e4m3_kernel(const uint8_t *__restrict__ codes, int64_t numel,
                                                       uint16_t *__restrict__ out, int out_bf16, int vec_ok) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  auto one = [&](uint8_t c) -> uint16_t {
    __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E4M3);
    if (!out_bf16) return h.x;
    return __bfloat16_as_ushort(__float2bfloat16_rn(__half2float(__half(h))));
  };
  if (vec_ok) {
    const int64_t nvec = numel / 16;
    const uint4 *cv = reinterpret_cast<const uint4 *>(codes);
    uint4 *ov = reinterpret_cast<uint4 *>(out);
    for (int64_t i = tid; i < nvec; i += stride) {
      uint4 q = cv[i];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      uint32_t o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[2 * j] = one(w[j] & 0xff) | (static_cast<uint32_t>(one((w[j] >> 8) & 0xff)) << 16);
        o[2 * j + 1] = one((w[j] >> 16) & 0xff) | (static_cast<uint32_t>(one(w[j] >> 24)) << 16);
      }
      ov[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
      ov[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
    for (int64_t i = nvec * 16 + tid; i < numel; i += stride) out[i] = one(codes[i]);
  } else {
    for (int64_t i = tid; i < numel; i += stride) out[i] = one(codes[i]);
  }
}

struct ExpandDims {
  int ndim;
  int32_t shape[8];
  int64_t stride[8];
};

__global__ void __launch_bounds__(256) expand_16_kernel(const uint16_t *__restrict__ src, ExpandDims d, int64_t numel,
                                                      uint16_t *__restrict__ dst) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, off = 0;
    for (int a = d.ndim - 1; a >= 0; --a) {
      off += (rem % d.shape[a]) * d.stride[a];
      rem /= d.shape[a];
    }
    dst[i] = src[off];
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int capped_grid(int64_t work_items, int per_block) {
  int64_t g = (work_items + per_block - 1) / per_block;
  const int64_t cap = 148 * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace

int64_t helper_launch_count() { return g_helper_launches.load(); }

cudaError_t quantize_fp8_act(const void *x, int is_bf16, int m, int k, uint8_t *codes, float *scales,
                             cudaStream_t stream) {
  const bool vec = aligned16(x) && aligned16(codes) && (k % 16 == 0);
  const uint16_t *xs = static_cast<const uint16_t *>(x);
  // Launched behind the previous kernel in the stream with programmatic serialization, so that
  // its blocks are resident and waiting when that kernel's results become visible.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(m), 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (vec && k <= 2048 * 8) {
    cfg.blockDim = dim3(256, 1, 1);
    if (k <= 2048 * 2) e = cudaLaunchKernelEx(&cfg, quantize_fp8_act_reg_kernel<2>, xs, is_bf16, k, codes, scales);
    else if (k <= 2048 * 4) e = cudaLaunchKernelEx(&cfg, quantize_fp8_act_reg_kernel<4>, xs, is_bf16, k, codes, scales);
    else if (k <= 2048 * 6) e = cudaLaunchKernelEx(&cfg, quantize_fp8_act_reg_kernel<6>, xs, is_bf16, k, codes, scales);
    else e = cudaLaunchKernelEx(&cfg, quantize_fp8_act_reg_kernel<8>, xs, is_bf16, k, codes, scales);
  } else {
    cfg.blockDim = dim3(128, 1, 1);
    if (vec) e = cudaLaunchKernelEx(&cfg, quantize_fp8_act_kernel<true>, xs, is_bf16, k, codes, scales);
    else e = cudaLaunchKernelEx(&cfg, quantize_fp8_act_kernel<false>, xs, is_bf16, k, codes, scales);
  }
  ++g_helper_launches;
  return e;
}

cudaError_t quantize_fp8_scatter(const void *x, int is_bf16, int m, int k, const float *amax, uint8_t *const *dests,
                                 int n_dest, int64_t ld, int col0, float *scales, cudaStream_t stream) {
  if (n_dest < 1 || n_dest > 8 || k % 16 != 0 || ld % 16 != 0 || col0 % 16 != 0 || !aligned16(x)) return cudaErrorInvalidValue;
  ScatterDests d = {};
  d.count = n_dest;
  for (int i = 0; i < n_dest; ++i) {
    if (!aligned16(dests[i])) return cudaErrorInvalidValue;
    d.ptr[i] = dests[i];
  }
  quantize_fp8_scatter_kernel<<<static_cast<unsigned>(m), 128, 0, stream>>>(static_cast<const uint16_t *>(x), is_bf16, k, amax, d,
                                                                            ld, col0, scales);
  ++g_helper_launches;
  return cudaGetLastError();
}

cudaError_t row_amax_16(const void *x, int is_bf16, int m, int k, int64_t pitch, float *amax, cudaStream_t stream) {
  row_amax_kernel<<<static_cast<unsigned>(m), 128, 0, stream>>>(static_cast<const uint16_t *>(x), is_bf16, k, pitch, amax);
  ++g_helper_launches;
  return cudaGetLastError();
}

cudaError_t ln_modulate_quantize_fp8(const void *x, int is_bf16, int m, int k, const void *scale, int64_t scale_pitch,
                                     const void *shift, int64_t shift_pitch, int rows_per_group, float eps,
                                     uint8_t *codes, float *row_scales, cudaStream_t stream) {
  const bool vec = aligned16(x) && aligned16(codes) && (k % 8 == 0) && aligned16(scale) && aligned16(shift) &&
                   scale_pitch % 8 == 0 && shift_pitch % 8 == 0;
  const uint16_t *xs = static_cast<const uint16_t *>(x);
  const uint16_t *sc = static_cast<const uint16_t *>(scale);
  const uint16_t *sh = static_cast<const uint16_t *>(shift);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(m), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (vec && is_bf16 && k <= 1024 * 3) {
    cfg.blockDim = dim3(128, 1, 1);
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_bf16_kernel<3, 128>, xs, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  } else if (vec && is_bf16 && k <= 2048 * 2) {
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_bf16_kernel<2, 256>, xs, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  } else if (vec && is_bf16 && k <= 2048 * 4) {
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_bf16_kernel<4, 256>, xs, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  } else if (vec && k <= 1024 * 3) {
    cfg.blockDim = dim3(128, 1, 1);
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_reg_kernel<3, 128>, xs, is_bf16, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  } else if (vec && k <= 2048 * 2) {
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_reg_kernel<2, 256>, xs, is_bf16, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  } else if (vec && k <= 2048 * 4) {
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_reg_kernel<4, 256>, xs, is_bf16, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  } else if (vec && k <= 2048 * 8) {
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_reg_kernel<8, 256>, xs, is_bf16, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  } else {
    e = cudaLaunchKernelEx(&cfg, ln_modulate_quantize_kernel, xs, is_bf16, k, sc, sh, rows_per_group, scale_pitch, shift_pitch, eps, codes, row_scales);
  }
  ++g_helper_launches;
  return e;
}

cudaError_t swiglu_quantize_fp8(const void *x, int is_bf16, int m, int h, uint8_t *codes, float *row_scales,
                                cudaStream_t stream) {
  const bool vec = aligned16(x) && aligned16(codes) && (h % 8 == 0);
  const uint16_t *xs = static_cast<const uint16_t *>(x);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(m), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (vec && h <= 2048 * 2) {
    e = cudaLaunchKernelEx(&cfg, swiglu_quantize_reg_kernel<2>, xs, is_bf16, h, codes, row_scales);
  } else if (vec && h <= 2048 * 4) {
    e = cudaLaunchKernelEx(&cfg, swiglu_quantize_reg_kernel<4>, xs, is_bf16, h, codes, row_scales);
  } else if (vec && h <= 2048 * 7) {
    e = cudaLaunchKernelEx(&cfg, swiglu_quantize_reg_kernel<7>, xs, is_bf16, h, codes, row_scales);
  } else {
    e = cudaLaunchKernelEx(&cfg, swiglu_quantize_kernel, xs, is_bf16, h, codes, row_scales);
  }
  ++g_helper_launches;
  return e;
}

cudaError_t quantize_fp8_rows_f32(const float *w, int rows, int k, uint8_t *codes, float *scales,
                                  cudaStream_t stream) {
  quantize_fp8_rows_f32_kernel<<<rows, 128, 0, stream>>>(w, k, codes, scales);
  ++g_helper_launches;
  return cudaGetLastError();
}

cudaError_t quantize_nvfp4_act(const void *x, int is_bf16, int m, int k, uint8_t *codes, uint8_t *sf_tiled,
                               cudaStream_t stream) {
  const int64_t blocks = static_cast<int64_t>(m) * (k / 16);
  const int grid = static_cast<int>((blocks + 255) / 256);
  const int vec = aligned16(x) && (reinterpret_cast<uintptr_t>(codes) & 7) == 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, quantize_nvfp4_act_kernel, static_cast<const uint16_t *>(x), is_bf16, m, k, codes,
                                     sf_tiled, sf_k_tiles_for(k), vec);
  ++g_helper_launches;
  return e;
}

cudaError_t nvfp4_prepare(const void *x, int is_bf16, int m, int k, uint8_t *codes, uint8_t *sfa_tiled,
                          const uint8_t *wsf_plain, int rows, int w_extra_groups, uint8_t *sfb_tiled, cudaStream_t stream) {
  const int sf_k_tiles = sf_k_tiles_for(k);
  const int64_t a_threads = static_cast<int64_t>((m + 127) / 128) * 128 * sf_k_tiles * 4;
  const int w_groups = (rows + 127) / 128 + w_extra_groups;
  const int64_t b_threads = static_cast<int64_t>(w_groups) * 128 * sf_k_tiles;
  const int a_ctas = static_cast<int>((a_threads + 255) / 256), b_ctas = static_cast<int>((b_threads + 255) / 256);
  const int vec = aligned16(x) && (reinterpret_cast<uintptr_t>(codes) & 7) == 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(a_ctas + b_ctas), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, nvfp4_prepare_kernel, static_cast<const uint16_t *>(x), is_bf16, m, k, codes,
                                     sfa_tiled, sf_k_tiles, vec, a_ctas, wsf_plain, rows, w_groups, sfb_tiled);
  ++g_helper_launches;
  return e;
}

cudaError_t quantize_nvfp4_weight_f32(const float *w, int rows, int k, uint8_t *codes, uint8_t *sf_plain,
                                      float *global_scale, uint32_t *amax_word, cudaStream_t stream) {
  const int64_t numel = static_cast<int64_t>(rows) * k;
  cudaError_t e = cudaMemsetAsync(amax_word, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return e;
  amax_f32_kernel<<<capped_grid(numel, 256 * 8), 256, 0, stream>>>(w, numel, amax_word);
  nvfp4_global_scale_kernel<<<1, 1, 0, stream>>>(amax_word, global_scale);
  const int64_t blocks = numel / 16;
  quantize_nvfp4_weight_kernel<<<static_cast<int>((blocks + 255) / 256), 256, 0, stream>>>(w, rows, k, global_scale,
                                                                                          codes, sf_plain);
  g_helper_launches += 3;
  return cudaGetLastError();
}

cudaError_t pack_scale_factors(const uint8_t *sf_plain, int rows, int k, uint8_t *sf_tiled, cudaStream_t stream) {
  const int kblocks = k / 16;
  const int64_t n = static_cast<int64_t>(rows) * kblocks;
  pack_sf_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, stream>>>(sf_plain, rows, kblocks, sf_tiled,
                                                                       sf_k_tiles_for(k));
  ++g_helper_launches;
  return cudaGetLastError();
}

cudaError_t widen_e4m3(const uint8_t *codes, int64_t numel, void *out16, int out_bf16, cudaStream_t stream) {
  const int vec = aligned16(codes) && aligned16(out16);
  widen_e4m3_kernel<<<capped_grid(numel, 256 * 16), 256, 0, stream>>>(codes, numel, static_cast<uint16_t *>(out16),
                                                                     out_bf16, vec);
  ++g_helper_launches;
  return cudaGetLastError();
}

cudaError_t expand_16(const void *src, const int32_t *shape, const int64_t *stride, int ndim, void *dst,
                      cudaStream_t stream) {
  if (ndim > 8) return cudaErrorInvalidValue;
  ExpandDims d;
  d.ndim = ndim;
  int64_t numel = 1;
  for (int i = 0; i < ndim; ++i) {
    d.shape[i] = shape[i];
    d.stride[i] = stride[i];
    numel *= shape[i];
  }
  if (numel == 0) return cudaSuccess;
  expand_16_kernel<<<capped_grid(numel, 256), 256, 0, stream>>>(static_cast<const uint16_t *>(src), d, numel,
                                                               static_cast<uint16_t *>(dst));
  ++g_helper_launches;
  return cudaGetLastError();
}

}  // namespace flsm100
