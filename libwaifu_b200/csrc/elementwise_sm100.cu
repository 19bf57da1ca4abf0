// copy / cast / fill / add over float, half and bfloat16 views (flint/capi.h:246-249,279,483;
// the reference's kernels are flint/cuda/copy.cu, cast.cu, fill.cu, binary.cu). Contiguous,
// 16-byte aligned operands take a vector path (eight elements per thread per step, grid-stride
// over a grid of a few CTAs per SM); anything else goes through a per-element path that walks
// the views' strides. Sums are taken in fp32 and rounded once, which for 16-bit operands is the
// same value the reference's half arithmetic gives (the sum of two halves is exact in fp32).
#include "elementwise_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "gemm_sm100.cuh"

namespace flsm100 {

namespace {

std::atomic<int64_t> g_elem_launches{0};

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;

__device__ __forceinline__ float load1(const void *p, int kind, int64_t i) {
  if (kind == kElemF32) return reinterpret_cast<const float *>(p)[i];
  const uint16_t v = reinterpret_cast<const uint16_t *>(p)[i];
  if (kind == kElemBF16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  return __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ void store1(void *p, int kind, int64_t i, float v) {
  if (kind == kElemF32) {
    reinterpret_cast<float *>(p)[i] = v;
  } else if (kind == kElemBF16) {
    reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
  } else {
    reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
  }
}

// Eight consecutive elements starting at element i (a multiple of 8) of a 16-byte aligned base.
__device__ __forceinline__ void load8(const void *p, int kind, int64_t i, float (&v)[8]) {
  if (kind == kElemF32) {
    const float4 lo = reinterpret_cast<const float4 *>(p)[i / 4];
    const float4 hi = reinterpret_cast<const float4 *>(p)[i / 4 + 1];
    v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
    return;
  }
  const uint4 q = reinterpret_cast<const uint4 *>(p)[i / 8];
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (kind == kElemBF16) {
      v[2 * j] = __uint_as_float(w[j] << 16);
      v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
      v[2 * j] = f.x, v[2 * j + 1] = f.y;
    }
  }
}

__device__ __forceinline__ void store8(void *p, int kind, int64_t i, const float (&v)[8]) {
  if (kind == kElemF32) {
    reinterpret_cast<float4 *>(p)[i / 4] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(p)[i / 4 + 1] = make_float4(v[4], v[5], v[6], v[7]);
    return;
  }
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (kind == kElemBF16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t *>(&h);
    } else {
      const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
  }
  reinterpret_cast<uint4 *>(p)[i / 8] = make_uint4(w[0], w[1], w[2], w[3]);
}

// Strides of up to three operands over one shape.
struct Walk {
  int ndim;
  int32_t shape[kMaxElemDims];
  int64_t s0[kMaxElemDims], s1[kMaxElemDims], s2[kMaxElemDims];
};

__device__ __forceinline__ void offsets(const Walk &w, int64_t idx, int64_t *o0, int64_t *o1, int64_t *o2) {
  int64_t a = 0, b = 0, c = 0;
#pragma unroll
  for (int d = kMaxElemDims - 1; d >= 0; --d) {
    if (d < w.ndim) {
      const int64_t q = idx / w.shape[d];
      const int64_t r = idx - q * w.shape[d];
      a += r * w.s0[d], b += r * w.s1[d], c += r * w.s2[d];
      idx = q;
    }
  }
  *o0 = a, *o1 = b, *o2 = c;
}

// OP 0: out = in (cast or copy through fp32); 1: out = a + b; 2: out = value.
template <int OP>
__global__ void __launch_bounds__(kThreads) vector_kernel(const void *a, int a_kind, const void *b, void *out, int out_kind,
                                                          int64_t numel, float value) {
  const int64_t groups = numel / 8;
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += step) {
    float x[8];
    if (OP == 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = value;
    } else {
      load8(a, a_kind, g * 8, x);
      if (OP == 1) {
        float y[8];
        load8(b, a_kind, g * 8, y);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __fadd_rn(x[j], y[j]);
      }
    }
    store8(out, out_kind, g * 8, x);
  }
  // the last numel % 8 elements, one thread each
  const int64_t tail0 = groups * 8;
  const int64_t t = tail0 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < numel) {
    float x = value;
    if (OP != 2) {
      x = load1(a, a_kind, t);
      if (OP == 1) x = __fadd_rn(x, load1(b, a_kind, t));
    }
    store1(out, out_kind, t, x);
  }
}

template <int OP>
__global__ void __launch_bounds__(kThreads) strided_kernel(const void *a, int a_kind, const void *b, void *out, int out_kind,
                                                           Walk w, int64_t numel, float value) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel; i += step) {
    int64_t oa, ob, oo;
    offsets(w, i, &oa, &ob, &oo);
    float x = value;
    if (OP != 2) {
      x = load1(a, a_kind, oa);
      if (OP == 1) x = __fadd_rn(x, load1(b, a_kind, ob));
    }
    store1(out, out_kind, oo, x);
  }
}

// Raw elements of 1, 2, 4 or 8 bytes moved between two strided views.
template <typename T>
__global__ void __launch_bounds__(kThreads) copy_strided_kernel(const T *in, T *out, Walk w, int64_t numel) {
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < numel; i += step) {
    int64_t oi, unused, oo;
    offsets(w, i, &oi, &unused, &oo);
    out[oo] = in[oi];
  }
}

int grid_for(int64_t work_items) {
  int64_t blocks = (work_items + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * kCtasPerSm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

Walk make_walk(const ElemView *v0, const ElemView *v1, const ElemView *v2) {
  Walk w = {};
  w.ndim = v0->ndim;
  for (int d = 0; d < v0->ndim; ++d) {
    w.shape[d] = v0->shape[d];
    w.s0[d] = v0->stride[d];
    w.s1[d] = v1 ? v1->stride[d] : 0;
    w.s2[d] = v2 ? v2->stride[d] : 0;
  }
  return w;
}

template <int OP>
cudaError_t run(const ElemView *a, int a_kind, const ElemView *b, const ElemView &out, int out_kind, int64_t numel,
                float value, cudaStream_t stream) {
  if (numel <= 0) return cudaSuccess;
  const bool vec = out.contiguous && aligned16(out.base) && (!a || (a->contiguous && aligned16(a->base))) &&
                   (!b || (b->contiguous && aligned16(b->base)));
  if (vec) {
    vector_kernel<OP><<<grid_for((numel + 7) / 8), kThreads, 0, stream>>>(a ? a->base : nullptr, a_kind, b ? b->base : nullptr,
                                                                          const_cast<void *>(out.base), out_kind, numel, value);
  } else {
    const Walk w = make_walk(a ? a : &out, b, &out);
    strided_kernel<OP><<<grid_for(numel), kThreads, 0, stream>>>(a ? a->base : nullptr, a_kind, b ? b->base : nullptr,
                                                                  const_cast<void *>(out.base), out_kind, w, numel, value);
  }
  ++g_elem_launches;
  return cudaGetLastError();
}

}  // namespace

cudaError_t elementwise_cast(const ElemView &in, ElemKind in_kind, const ElemView &out, ElemKind out_kind, int64_t numel,
                             cudaStream_t stream) {
  return run<0>(&in, in_kind, nullptr, out, out_kind, numel, 0.0f, stream);
}

cudaError_t elementwise_fill(const ElemView &view, ElemKind kind, int64_t numel, float value, cudaStream_t stream) {
  return run<2>(nullptr, kind, nullptr, view, kind, numel, value, stream);
}

cudaError_t elementwise_add(const ElemView &a, const ElemView &b, const ElemView &out, ElemKind kind, int64_t numel,
                            cudaStream_t stream) {
  return run<1>(&a, kind, &b, out, kind, numel, 0.0f, stream);
}

cudaError_t elementwise_copy(const ElemView &in, const ElemView &out, int bytes, int64_t numel, cudaStream_t stream) {
  if (numel <= 0) return cudaSuccess;
  if (in.contiguous && out.contiguous) {
    return cudaMemcpyAsync(const_cast<void *>(out.base), in.base, static_cast<size_t>(numel) * bytes,
                           cudaMemcpyDeviceToDevice, stream);
  }
  const Walk w = make_walk(&in, nullptr, &out);
  const int grid = grid_for(numel);
  void *o = const_cast<void *>(out.base);
  switch (bytes) {
    case 1: copy_strided_kernel<uint8_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint8_t *>(in.base), static_cast<uint8_t *>(o), w, numel); break;
    case 2: copy_strided_kernel<uint16_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint16_t *>(in.base), static_cast<uint16_t *>(o), w, numel); break;
    case 4: copy_strided_kernel<uint32_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint32_t *>(in.base), static_cast<uint32_t *>(o), w, numel); break;
    case 8: copy_strided_kernel<uint64_t><<<grid, kThreads, 0, stream>>>(static_cast<const uint64_t *>(in.base), static_cast<uint64_t *>(o), w, numel); break;
    default: return cudaErrorInvalidValue;
  }
  ++g_elem_launches;
  return cudaGetLastError();
}

int64_t elementwise_launch_count() { return g_elem_launches.load(); }

}  // namespace flsm100
