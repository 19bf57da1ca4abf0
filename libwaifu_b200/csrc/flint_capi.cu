// The C ABI of libflint_sm100.so (declared in include/flint_sm100.h): handles, the thread-local
// error, the argument checks of flint's FP8 entry points (flint/capi.cc:955-1097) restated, and
// the dispatch into the sm_100a kernels. There is no CPU path: a call that cannot run on the GPU
// fails with an error code.
#include "../../include/flint_sm100.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "gemm_sm100.cuh"
#include "quant_sm100.cuh"
#include "block_sm100.cuh"
#include "skinny_sm100.cuh"
#include "attention_sm100.cuh"
#include "elementwise_sm100.cuh"
#include "fewrow_tc_sm100.cuh"
#include "peer_sm100.cuh"
#include "selftest_sm100.cuh"
#include "matmul_simt_sm100.cuh"

using namespace flsm100;

struct fl_tensor_data_impl_t {
  void *ptr = nullptr;
  int64_t numel = 0;
  fl_dtype_t dtype = FL_DTYPE_UNKNOWN;
  fl_device_type_t device = FL_DEVICE_UNKNOWN;
  bool owned = false;
  bool ipc_mapped = false;  // another process's device storage, opened through its IPC handle
  // Device storage from the stream-ordered pool is given back in the order of the stream that
  // last owned its bytes (flint/cuda/cuda_tensor_data.cc:62-77); `resident` storage is a weight's
  // own cudaMalloc (flint/cuda/cuda_tensor_data.cc:44-48) and the only kind that can be exported.
  bool pooled = false;
  bool resident = false;
  cudaStream_t stream = nullptr;
  // The stream a pooled block was taken on when that is not the compute stream (an upload's
  // destination is taken on the copy stream): it goes back in that stream's order, behind the
  // compute stream's last use, so that the next upload finds it free without the pool growing.
  cudaStream_t home = nullptr;
};

// flint/capi.cc:530-535: the event that marks the end of a copy, and the storage it fills.
struct fl_transfer_impl_t {
  cudaEvent_t event = nullptr;
  fl_tensor_data_impl_t *dest = nullptr;  // null for a copy towards the host
};

struct fl_tensor_view_impl_t {
  fl_tensor_data_impl_t *data = nullptr;
  std::vector<int32_t> shape;
  std::vector<int32_t> stride;
  int64_t offset = 0;
};

struct fl_operators_impl_t {
  fl_device_type_t device;
};

namespace {

// ---- errors ------------------------------------------------------------------------------

struct FlError {
  int32_t code;
  std::string message;
};

[[noreturn]] void invalid(const std::string &m) { throw FlError{FL_ERROR_INVALID_ARG, m}; }
[[noreturn]] void aborted(const std::string &m) { throw FlError{FL_ERROR_ABORTED, m}; }

thread_local int32_t t_code = FL_OK;
thread_local std::string t_message;

int32_t set_error(int32_t code, const std::string &message) {
  t_code = code;
  t_message = message;
  return code;
}

int32_t clear_error() {
  t_code = FL_OK;
  t_message.clear();
  return FL_OK;
}

// Runs `body`; whatever it throws becomes an error code (flint/capi.cc:191-206).
template <typename Body>
int32_t guard(Body &&body) {
  try {
    return body();
  } catch (const FlError &e) {
    return set_error(e.code, e.message);
  } catch (const std::bad_alloc &) {
    return set_error(FL_ERROR_ABORTED, "out of memory");
  } catch (const std::exception &e) {
    return set_error(FL_ERROR_ABORTED, e.what());
  } catch (...) {
    return set_error(FL_ERROR_ABORTED, "unknown exception");
  }
}

void cuda_check(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return;
  std::string m = std::string(what) + ": " + cudaGetErrorString(e);
  if (e == cudaErrorMemoryAllocation) throw FlError{FL_ERROR_OUT_OF_MEMORY, m};
  aborted(m);
}

// ---- dtypes ------------------------------------------------------------------------------

int64_t dtype_size(fl_dtype_t t) {
  switch (t) {
    case FL_DTYPE_FLOAT: return 4;
    case FL_DTYPE_LONG: return 8;
    case FL_DTYPE_UINT8: return 1;
    case FL_DTYPE_FLOAT16: return 2;
    case FL_DTYPE_INT8: return 1;
    case FL_DTYPE_BOOL: return 1;
    case FL_DTYPE_INT32: return 4;
    case FL_DTYPE_FP8E4M3: return 1;
    case FL_DTYPE_BFLOAT16: return 2;
    case FL_DTYPE_FP4E2M1X2: return 1;
    default: invalid("unknown dtype");
  }
}

const char *device_name(fl_device_type_t d) {
  switch (d) {
    case FL_DEVICE_CPU: return "cpu";
    case FL_DEVICE_CUDA: return "cuda";
    case FL_DEVICE_CUDA_HOST: return "cuda_host";
    case FL_DEVICE_METAL: return "metal";
    case FL_DEVICE_VULKAN: return "vulkan";
    default: return "unknown";
  }
}

// ---- the device --------------------------------------------------------------------------

struct DeviceState {
  bool probed = false;
  bool present = false;  // a CUDA device exists
  bool sm100 = false;    // and it is compute capability 10.x
  // Kernel status word in mapped host memory: kernels write it, the host reads it without a copy.
  uint32_t *status_host = nullptr;
  uint32_t *status_dev = nullptr;
  // Grow-only scratch for quantised activations, re-tiled scale factors and widened weights: one
  // block of the stream-ordered pool. All work is ordered on the legacy default stream, so it can be
  // reused call after call.
  uint8_t *scratch = nullptr;
  size_t scratch_cap = 0;
  // Set by the first call that touches the GPU: from then on this process belongs to that device
  // (per-process caches in the kernel modules assume one), and fl_sm100_set_device() refuses another.
  int device_in_use = -1;
  bool pool_ready = false;
  // Non-blocking streams the asynchronous transfers run on (flint/cuda/copy_stream.cc:31), one
  // per direction so that uploads and downloads share the full-duplex link.
  cudaStream_t upload_stream = nullptr;
  cudaStream_t download_stream = nullptr;
  // Workspace of the GEMM's stream-K schedule: accumulator parts and the counters beside them
  // (zero between launches). Made once, on the first GEMM, and kept.
  float *sk_partials = nullptr;
  uint32_t *sk_counters = nullptr;
  // Upload destinations on their way back to the pool: a block taken on the copy stream goes back
  // in that stream's order (so that the next upload reuses it at once), but only after the compute
  // stream's last use of it has completed, which `used` marks; nothing waits, the list is swept
  // at the next upload or release.
  struct Returning {
    void *ptr;
    cudaEvent_t used;
    cudaStream_t home;
  };
  std::vector<Returning> returning;
};

std::mutex g_mutex;
DeviceState g_dev;

// Gives back every block of the list whose last use has completed (all of them when `all`: the
// caller has synchronised the compute stream). Called with g_mutex held.
void sweep_returning_locked(bool all) {
  size_t kept = 0;
  for (size_t i = 0; i < g_dev.returning.size(); ++i) {
    DeviceState::Returning r = g_dev.returning[i];
    if (all || cudaEventQuery(r.used) == cudaSuccess) {
      cudaEventDestroy(r.used);
      cudaFreeAsync(r.ptr, r.home);
    } else {
      g_dev.returning[kept++] = r;
    }
  }
  cudaGetLastError();  // cudaErrorNotReady from a query is not an error of ours
  g_dev.returning.resize(kept);
}
std::atomic<int64_t> g_gemm_launches{0};
std::atomic<int64_t> g_block_launches{0};  // kernels of block_sm100.cu

// Optional per-launch timing of the GEMM kernel alone (events on the launching stream), so a
// benchmark can separate it from the quantisation kernels launched by the same entry point.
struct GemmTiming {
  bool enabled = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> used;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> spare;
};
GemmTiming g_timing;

void probe_locked() {
  if (g_dev.probed) return;
  g_dev.probed = true;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count < 1) {
    cudaGetLastError();
    return;
  }
  g_dev.present = true;
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess) {
    g_dev.sm100 = (major == 10);
  }
}

DeviceState &device_state() {
  std::lock_guard<std::mutex> lock(g_mutex);
  probe_locked();
  return g_dev;
}

void require_kernels() {
  DeviceState &d = device_state();
  if (!d.present) aborted("no CUDA device is present");
  if (!d.sm100) aborted("the CUDA device is not compute capability 10.x; these kernels are sm_100a only");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (d.device_in_use < 0) {
    int dev = 0;
    cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
    d.device_in_use = dev;
  }
}

// The stream-ordered pool every activation and temporary comes from: the device's default pool,
// told to keep what is freed instead of handing it back to the driver at the next
// synchronisation (flint/cuda/cuda_operators.cc:91-98).
void ensure_pool() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_dev.pool_ready) return;
  int dev = 0;
  cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
  int supported = 0;
  cuda_check(cudaDeviceGetAttribute(&supported, cudaDevAttrMemoryPoolsSupported, dev), "cudaDeviceGetAttribute");
  if (!supported) aborted("the CUDA device does not support stream-ordered memory allocation");
  cudaMemPool_t pool;
  uint64_t threshold = UINT64_MAX;
  cuda_check(cudaDeviceGetDefaultMemPool(&pool, dev), "cudaDeviceGetDefaultMemPool");
  cuda_check(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold), "cudaMemPoolSetAttribute");
  // One contiguous reserve to start from (FLINT_SM100_POOL_RESERVE_MB, default 1024, 0 for none):
  // a pool that has grown piece by piece serves a 30 MB block by mapping more memory even when it
  // holds enough in pieces, which costs tens of microseconds a call and, now and then, tens of
  // milliseconds; taken and given back once, the reserve stays with the pool.
  size_t reserve_mb = 1024;
  if (const char *e = std::getenv("FLINT_SM100_POOL_RESERVE_MB")) reserve_mb = static_cast<size_t>(std::strtoull(e, nullptr, 10));
  if (reserve_mb > 0) {
    void *p = nullptr;
    if (cudaMallocAsync(&p, reserve_mb << 20, 0) == cudaSuccess) {
      cudaFreeAsync(p, 0);
    } else {
      cudaGetLastError();  // a card too full for the reserve runs without it
    }
  }
  g_dev.pool_ready = true;
}

cudaStream_t copy_stream(bool upload) {
  std::lock_guard<std::mutex> lock(g_mutex);
  cudaStream_t &st = upload ? g_dev.upload_stream : g_dev.download_stream;
  if (!st) cuda_check(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
  return st;
}

uint32_t *status_word() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_dev.status_host) {
    void *h = nullptr;
    cuda_check(cudaHostAlloc(&h, 64, cudaHostAllocMapped), "cudaHostAlloc(status)");
    std::memset(h, 0, 64);
    void *d = nullptr;
    cuda_check(cudaHostGetDevicePointer(&d, h, 0), "cudaHostGetDevicePointer(status)");
    g_dev.status_host = static_cast<uint32_t *>(h);
    g_dev.status_dev = static_cast<uint32_t *>(d);
  }
  return g_dev.status_dev;
}

// The status word of fl_fp8_linear_static()'s kernels, which lives in that entry point's fixed
// device array: read back and cleared (4 bytes each way, no allocation) once the array's address
// has been looked up on this device, 0 before. The caller has synchronised the stream.
uint32_t take_static_status();

// A GEMM that gave up on a wait may have left some of the stream-K counters counted up.
void rezero_stream_k_counters() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_dev.sk_counters) cudaMemsetAsync(g_dev.sk_counters, 0, gemm_stream_k_counter_words() * sizeof(uint32_t), 0);
}

// A kernel that gave up on a wait in an earlier call is reported by the next call.
void check_earlier_kernel_status() {
  uint32_t *h;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    h = g_dev.status_host;
  }
  if (h && *reinterpret_cast<volatile uint32_t *>(h) != 0) {
    uint32_t code = *reinterpret_cast<volatile uint32_t *>(h);
    *reinterpret_cast<volatile uint32_t *>(h) = 0;
    rezero_stream_k_counters();
    aborted("an earlier kernel gave up on a bounded wait (status " + std::to_string(code) + ")");
  }
}

// Bump allocation out of the scratch arena; `reset` at the start of every entry point.
struct Scratch {
  size_t used = 0;
  std::vector<std::pair<size_t, size_t>> wants;  // (offset, bytes)

  size_t reserve(size_t bytes) {
    size_t off = (used + 255) & ~size_t(255);
    used = off + bytes;
    return off;
  }
  // Grows the arena if needed (a rare event) and returns its base. The old block goes back to the
  // pool and the new one comes from it in stream 0's order (flint's temporaries do the same through
  // llynCudaAlloc, flint/cuda/common.h:197-202), so growing does not make the host or the device wait:
  // kernels already queued keep the old block until the stream reaches the free.
  uint8_t *commit() {
    if (used > g_dev.scratch_cap) ensure_pool();
    std::lock_guard<std::mutex> lock(g_mutex);
    if (used > g_dev.scratch_cap) {
      size_t cap = used + used / 4 + (1 << 20);
      if (g_dev.scratch) {
        cuda_check(cudaFreeAsync(g_dev.scratch, 0), "cudaFreeAsync(scratch)");
        g_dev.scratch = nullptr;
        g_dev.scratch_cap = 0;
      }
      void *p = nullptr;
      cuda_check(cudaMallocAsync(&p, cap, 0), "cudaMallocAsync(scratch)");
      g_dev.scratch = static_cast<uint8_t *>(p);
      g_dev.scratch_cap = cap;
    }
    return g_dev.scratch;
  }
};

// ---- views -------------------------------------------------------------------------------

fl_tensor_data_impl_t &deref(fl_tensor_data_t d) {
  if (!d) invalid("tensor data is null");
  return *d;
}

fl_tensor_view_impl_t &deref(fl_tensor_view_t v) {
  if (!v) invalid("tensor view is null");
  return *v;
}

int64_t numel_of(const fl_tensor_view_impl_t &v) {
  int64_t n = 1;
  for (int32_t s : v.shape) n *= s;
  return n;
}

// flint/tensor_view.cc:163-170
bool is_contiguous(const fl_tensor_view_impl_t &v) {
  int64_t numel = 1;
  for (int i = static_cast<int>(v.shape.size()) - 1; i >= 0; --i) {
    if (numel != v.stride[i] && v.shape[i] != 1) return false;
    numel *= v.shape[i];
  }
  return true;
}

std::string shape_string(const std::vector<int32_t> &shape) {
  std::string s = "(";
  for (size_t i = 0; i < shape.size(); ++i) {
    if (i) s += ", ";
    s += std::to_string(shape[i]);
  }
  return s + ")";
}

uint8_t *raw_ptr(const fl_tensor_view_impl_t &v) {
  return static_cast<uint8_t *>(v.data->ptr) + v.offset * dtype_size(v.data->dtype);
}

fl_dtype_t dtype_of(const fl_tensor_view_impl_t &v) { return v.data->dtype; }
fl_device_type_t device_of(const fl_tensor_view_impl_t &v) { return v.data->device; }

constexpr int64_t kMaxStorageElements = int64_t(1) << 30;  // TensorData::MaxNumEl, flint/tensor.h:41
constexpr size_t kResidentWeightBytes = size_t(2) << 20;   // flint/cuda/common.h:167

bool is_half_type(fl_dtype_t t) { return t == FL_DTYPE_FLOAT16 || t == FL_DTYPE_BFLOAT16; }

bool elem_kind_of(fl_dtype_t t, ElemKind *kind) {
  switch (t) {
    case FL_DTYPE_FLOAT: *kind = kElemF32; return true;
    case FL_DTYPE_FLOAT16: *kind = kElemF16; return true;
    case FL_DTYPE_BFLOAT16: *kind = kElemBF16; return true;
    default: return false;
  }
}


void check_shape(const fl_tensor_view_impl_t &v, const std::vector<int32_t> &shape, const char *what) {
  if (v.shape != shape) {
    invalid(std::string(what) + " is " + shape_string(v.shape) + " where " + shape_string(shape) + " was expected");
  }
}

// ---- the checks of flint/capi.cc:979-1035, restated --------------------------------------

void check_fp8_weight(const fl_tensor_view_impl_t &data, const fl_tensor_view_impl_t &scale, bool per_channel_ok) {
  if (dtype_of(data) != FL_DTYPE_FP8E4M3 || data.shape.size() != 2) {
    invalid("fp8 operand: data is not <fp8e4m3>(rows, k)");
  }
  const int64_t sn = numel_of(scale);
  if (dtype_of(scale) != FL_DTYPE_FLOAT || !(sn == 1 || (per_channel_ok && sn == data.shape[0]))) {
    invalid(per_channel_ok ? "fp8 operand: the scale is not <float>(1) or <float>(rows)"
                           : "fp8 operand: the scale is not a single <float>");
  }
  if (device_of(data) != device_of(scale)) invalid("fp8 operand: the data and the scale are on different devices");
  if (!is_contiguous(data) || !is_contiguous(scale)) invalid("fp8 operand: not contiguous");
  if (numel_of(data) >= INT32_MAX) invalid("fp8 operand: more elements than the kernels can index");
}

void check_activation(const fl_tensor_view_impl_t &x, fl_device_type_t device, const char *what) {
  if (device_of(x) != device) invalid(std::string(what) + " is not on the same device as the weight");
  if (!is_contiguous(x)) invalid(std::string(what) + " is not contiguous");
  if (x.shape.size() < 2) invalid(std::string(what) + " has fewer than two dimensions");
  if (!is_half_type(dtype_of(x))) {
    invalid(std::string(what) + " is not <float16> (or <bfloat16>), which is what this device multiplies in");
  }
}

void check_result(const fl_tensor_view_impl_t &out, const fl_tensor_view_impl_t &a, int rows,
                  fl_device_type_t device) {
  if (device_of(out) != device || dtype_of(out) != dtype_of(a)) {
    invalid("out is not <float16> on the weight's device (or <bfloat16> where the left operand is)");
  }
  if (!is_contiguous(out)) invalid("out is not contiguous");
  std::vector<int32_t> shape = a.shape;
  shape.back() = rows;
  check_shape(out, shape, "out");
}

void check_tiles(int rows, int k, int k_multiple) {
  if (rows % 8 != 0) invalid("the fp8 operand's row count is not a multiple of 8");
  if (k % k_multiple != 0) {
    invalid("the " + std::string(k_multiple == 16 ? "fp8" : "nvfp4") + " operand's k is not a multiple of " +
            std::to_string(k_multiple));
  }
}

int64_t leading_rows(const fl_tensor_view_impl_t &a) {
  int64_t m = 1;
  for (size_t i = 0; i + 1 < a.shape.size(); ++i) m *= a.shape[i];
  return m;
}

// How the epilogue reads an addend: as a bias, as rows that repeat with a period over m, or (when
// neither fits) from an expanded copy in scratch.
struct AddendPlan {
  const void *bias = nullptr;
  const void *residual = nullptr;
  int residual_rows = 0;
  int64_t residual_ld = 0;
  bool needs_expand = false;
};

// `addend` broadcast over out's leading dimensions (right-aligned, each dimension 1 or equal).
AddendPlan plan_addend(const fl_tensor_view_impl_t &addend, const fl_tensor_view_impl_t &out,
                       std::vector<int32_t> *bshape, std::vector<int64_t> *bstride) {
  const int od = static_cast<int>(out.shape.size());
  const int ad = static_cast<int>(addend.shape.size());
  const int n = out.shape.back();
  if (ad < 1 || addend.shape.back() != n) invalid("the addend's last dimension is not out's");
  bshape->assign(out.shape.begin(), out.shape.end());
  bstride->assign(od, 0);
  for (int i = 0; i < ad; ++i) {
    const int o = od - ad + i;
    if (addend.shape[i] == out.shape[o]) {
      (*bstride)[o] = (addend.shape[i] == 1) ? 0 : addend.stride[i];
    } else if (addend.shape[i] == 1) {
      (*bstride)[o] = 0;
    } else {
      invalid("the addend does not broadcast over out's leading dimensions");
    }
  }
  AddendPlan plan;
  const void *base = raw_ptr(addend);
  const bool unit_last = (n == 1) || (*bstride)[od - 1] == 1;
  // Leading dimensions of extent 1 index nothing.
  bool all_leading_zero = true;
  for (int i = 0; i < od - 1; ++i) {
    if (out.shape[i] != 1 && (*bstride)[i] != 0) all_leading_zero = false;
  }
  if (unit_last && all_leading_zero) {
    plan.bias = base;  // (n), or a zero-stride expansion of it: read in the epilogue as a bias
    return plan;
  }
  if (unit_last) {
    // Rows with pitch L whose pattern repeats with period P over m: a suffix of the leading
    // dimensions dense with pitch L, everything before it broadcast.
    int i = od - 2;
    while (i >= 0 && out.shape[i] == 1) --i;
    if (i >= 0 && (*bstride)[i] >= n) {
      const int64_t ld = (*bstride)[i];
      int64_t period = 1;
      int64_t expect = ld;
      bool ok = true;
      int j = i;
      for (; j >= 0; --j) {
        if (out.shape[j] == 1) continue;
        if ((*bstride)[j] == expect) {
          period *= out.shape[j];
          expect *= out.shape[j];
        } else {
          break;
        }
      }
      for (; j >= 0; --j) {
        if (out.shape[j] != 1 && (*bstride)[j] != 0) ok = false;
      }
      if (ok && period <= INT32_MAX) {
        plan.residual = base;
        plan.residual_rows = static_cast<int>(period);
        plan.residual_ld = ld;
        return plan;
      }
    }
  }
  plan.needs_expand = true;
  return plan;
}

struct Epilogue {
  // Scatter form: the product is columns [out_col0, out_col0 + n) of matrices of pitch out_ld,
  // `extra_out` being the peers' copies.
  void *extra_out[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int num_extra_out = 0;
  int64_t out_ld = 0;
  int out_col0 = 0;
  const float *row_scale = nullptr;
  const float *col_scale = nullptr;
  int col_scale_scalar = 0;
  const float *global_scale = nullptr;
  const void *bias = nullptr;
  const void *residual = nullptr;
  int residual_rows = 0;
  int64_t residual_ld = 0;
  int act = 0;
  int rows_per_group = 0;
  float *row_amax = nullptr;
};

// Where the tensor-core few-row kernels (fewrow_tc_sm100.cu) measured faster than what a product
// would run on otherwise; the thresholds are measurements on a B200 over 1-64 rows, 3072-24576
// channels and 3072- and 12288-deep rows. Host arithmetic only: fl_sm100_few_rows_route reports
// them, so that the CPU tests pin them.
// fl_fp8_matmul[_add], half rows against an e4m3 weight (fewrow_tc_kernel):
bool fewrow_tc_route(int m, int rows, int k) {
  if (m > 64) return false;
  if (m > 16) return k >= 2048 && rows >= 3072;
  return k >= 2048 ? rows >= 8192 || (rows >= 6144 && m >= 2) || (rows >= 3072 && m >= 8)
                   : rows >= 16384 || (rows >= 12288 && m >= 4) || (rows >= 8192 && m >= 8);
}
// fl_matmul[_add], 16-bit rows against a 16-bit weight (fewrow_q8_kernel, kind::f16):
bool fewrow_w16_route(int m, int n, int k) {
  if (m > 64 || k < 2048) return false;
  return m > 32 ? n >= 16384 || (n >= 3072 && k <= 6144) : m >= 8 ? n >= 3072 : m >= 4 ? n >= 6144 : n >= 16384;
}
// fl_fp8_linear and its relatives, quantised rows against an e4m3 weight (fewrow_q8_kernel):
bool fewrow_q8_route(int m, int rows, int k) {
  if (m > 32 || k < 2048) return false;
  return m >= 4 ? rows >= 3072 : rows >= 8192;
}

// The stream-K workspace, from the pool in stream 0's order the first time a GEMM runs (38 MB on a
// 148-SM card), kept for the life of the process.
void stream_k_workspace(GemmArgs *g) {
  ensure_pool();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_dev.sk_partials) {
    void *parts = nullptr, *counters = nullptr;
    const size_t counter_bytes = gemm_stream_k_counter_words() * sizeof(uint32_t);
    cuda_check(cudaMallocAsync(&parts, gemm_stream_k_partial_floats() * sizeof(float), 0), "cudaMallocAsync(stream-K parts)");
    cudaError_t e = cudaMallocAsync(&counters, counter_bytes, 0);
    if (e == cudaSuccess) e = cudaMemsetAsync(counters, 0, counter_bytes, 0);
    if (e != cudaSuccess) {
      cudaFreeAsync(parts, 0);
      if (counters) cudaFreeAsync(counters, 0);
      cuda_check(e, "cudaMallocAsync(stream-K counters)");
    }
    g_dev.sk_partials = static_cast<float *>(parts);
    g_dev.sk_counters = static_cast<uint32_t *>(counters);
  }
  g->sk_partials = g_dev.sk_partials;
  g->sk_partial_floats = gemm_stream_k_partial_floats();
  g->sk_counters = g_dev.sk_counters;
  g->sk_counter_words = gemm_stream_k_counter_words();
}

void run_gemm(GemmKind kind, int m, int n, int k, const void *a, const void *b, const uint8_t *sfa,
              const uint8_t *sfb, const Epilogue &ep, int out_bf16, void *out, bool b_is_e4m3 = false) {
  GemmArgs g{};
  g.b_is_e4m3 = b_is_e4m3 ? 1 : 0;
  g.kind = kind;
  g.m = m;
  g.n = n;
  g.k = k;
  g.a = a;
  g.b = b;
  g.sfa = sfa;
  g.sfb = sfb;
  g.sf_k_tiles = (kind == kGemmNvf4) ? sf_k_tiles_for(k) : 0;
  g.row_scale = ep.row_scale;
  g.col_scale = ep.col_scale;
  g.col_scale_scalar = ep.col_scale_scalar;
  g.global_scale = ep.global_scale;
  g.bias = ep.bias;
  g.residual = ep.residual;
  g.residual_rows = ep.residual_rows;
  g.residual_ld = ep.residual_ld;
  g.act = ep.act;
  g.rows_per_group = ep.rows_per_group;
  g.row_amax = ep.row_amax;
  g.out_bf16 = out_bf16;
  g.out = out;
  for (int i = 0; i < 7; ++i) g.extra_out[i] = ep.extra_out[i];
  g.num_extra_out = ep.num_extra_out;
  g.out_ld = ep.out_ld;
  g.out_col0 = ep.out_col0;
  g.status = status_word();
  g.stream = 0;
  // FLINT_SM100_SINGLE_CTA=1 keeps every GEMM on the single-CTA kernel (for A/B measurements).
  static const bool single_cta = []() {
    const char *v = std::getenv("FLINT_SM100_SINGLE_CTA");
    return v && v[0] == '1';
  }();
  g.force_single_cta = single_cta ? 1 : 0;
  // FLINT_SM100_NO_STREAM_K=1 keeps every tile whole (for A/B measurements and the parity tests
  // that compare the two schedules).
  const char *no_sk = std::getenv("FLINT_SM100_NO_STREAM_K");
  g.no_stream_k = (no_sk && no_sk[0] == '1') ? 1 : 0;
  if (!g.no_stream_k) stream_k_workspace(&g);
  const char *no_st = std::getenv("FLINT_SM100_NO_STAGED_EPILOGUE");
  g.no_staged_out = (no_st && no_st[0] == '1') ? 1 : 0;
  const char *why = "";
  std::pair<cudaEvent_t, cudaEvent_t> ev{nullptr, nullptr};
  if (g_timing.enabled) {
    if (!g_timing.spare.empty()) {
      ev = g_timing.spare.back();
      g_timing.spare.pop_back();
    } else {
      cuda_check(cudaEventCreate(&ev.first), "cudaEventCreate");
      cuda_check(cudaEventCreate(&ev.second), "cudaEventCreate");
    }
    cuda_check(cudaEventRecord(ev.first, g.stream), "cudaEventRecord");
  }
  cudaError_t e = launch_gemm(g, &why);
  if (ev.first) {
    cudaEventRecord(ev.second, g.stream);
    g_timing.used.push_back(ev);
  }
  if (e != cudaSuccess) aborted(std::string("GEMM launch: ") + why + " (" + cudaGetErrorString(e) + ")");
  ++g_gemm_launches;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Resolves the optional addend/bias/residual views of an entry point into epilogue pointers,
// expanding into scratch what the epilogue cannot index. Scratch offsets are reserved in
// `scratch` first and resolved after commit(), hence the two phases.
struct AddendResolver {
  AddendPlan plan;
  std::vector<int32_t> bshape;
  std::vector<int64_t> bstride;
  size_t expand_off = 0;
  const fl_tensor_view_impl_t *view = nullptr;

  void prepare(const fl_tensor_view_impl_t *addend, const fl_tensor_view_impl_t &out, Scratch *scratch) {
    view = addend;
    if (!addend) return;
    plan = plan_addend(*addend, out, &bshape, &bstride);
    if (plan.needs_expand) expand_off = scratch->reserve(static_cast<size_t>(numel_of(out)) * 2);
  }
  void resolve(uint8_t *scratch_base, int m, int n, Epilogue *ep) {
    if (!view) return;
    if (plan.needs_expand) {
      void *dst = scratch_base + expand_off;
      cuda_check(expand_16(raw_ptr(*view), bshape.data(), bstride.data(), static_cast<int>(bshape.size()), dst, 0),
                 "expanding the addend");
      ep->residual = dst;
      ep->residual_rows = m;
      ep->residual_ld = n;
    } else if (plan.bias) {
      ep->bias = plan.bias;
    } else {
      ep->residual = plan.residual;
      ep->residual_rows = plan.residual_rows;
      ep->residual_ld = plan.residual_ld;
    }
  }
};

}  // namespace

// ============================ Part 1 ==========================================================

extern "C" {

void fl_init(void) {
  guard([&]() {
    device_state();
    return clear_error();
  });
}

int32_t fl_is_device_available(fl_device_type_t device, int32_t *out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    DeviceState &d = device_state();
    switch (device) {
      case FL_DEVICE_CPU: *out = 1; break;  // storage only
      case FL_DEVICE_CUDA:
      case FL_DEVICE_CUDA_HOST: *out = (d.present && d.sm100) ? 1 : 0; break;
      case FL_DEVICE_METAL:
      case FL_DEVICE_VULKAN: *out = 0; break;
      default: invalid("unknown device");
    }
    return clear_error();
  });
}

int32_t fl_get_last_error_code(void) { return t_code; }

const char *fl_get_last_error_message(void) { return t_message.c_str(); }

int32_t fl_operators_create(fl_device_type_t device, fl_operators_t *out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    if (device != FL_DEVICE_CUDA) {
      invalid(std::string("this library has operators for cuda only, not ") + device_name(device));
    }
    require_kernels();
    *out = new fl_operators_impl_t{device};
    return clear_error();
  });
}

void fl_operators_destroy(fl_operators_t operators) { delete operators; }

int32_t fl_operators_get_device(fl_operators_t operators, fl_device_type_t *out) {
  return guard([&]() {
    if (!operators) invalid("operators is null");
    if (!out) invalid("out is null");
    *out = operators->device;
    return clear_error();
  });
}

int32_t fl_tensor_data_create(fl_device_type_t device, fl_dtype_t dtype, int64_t numel, fl_alloc_hint_t hint,
                              fl_tensor_data_t *out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    if (numel < 1) invalid("storage holds at least one element");
    if (numel > kMaxStorageElements) invalid("too many elements");  // flint/tensor.h:41
    if (hint < FL_ALLOC_ACTIVATION || hint > FL_ALLOC_TEMPORARY_WEIGHT) invalid("unknown allocation hint");
    const size_t bytes = static_cast<size_t>(numel * dtype_size(dtype));
    void *p = nullptr;
    bool pooled = false, resident = false;
    switch (device) {
      case FL_DEVICE_CPU:
        if (posix_memalign(&p, 64, bytes < 64 ? 64 : bytes) != 0) throw FlError{FL_ERROR_OUT_OF_MEMORY, "host allocation failed"};
        break;
      case FL_DEVICE_CUDA:
        require_kernels();
        // flint/cuda/cuda_tensor_data.cc:36-52: a weight of 2 MiB or more gets memory of its own (it
        // stays until it is let go of, and then goes back to the driver whole); everything else
        // comes from the pool in stream 0's order, which makes neither the host nor the device wait.
        resident = hint == FL_ALLOC_WEIGHT && bytes >= kResidentWeightBytes;
        if (resident) {
          cuda_check(cudaMalloc(&p, bytes), "cudaMalloc");
        } else {
          ensure_pool();
          cuda_check(cudaMallocAsync(&p, bytes, 0), "cudaMallocAsync");
          pooled = true;
        }
        break;
      case FL_DEVICE_CUDA_HOST:
        require_kernels();
        cuda_check(cudaMallocHost(&p, bytes), "cudaMallocHost");
        break;
      default: invalid(std::string("no storage on ") + device_name(device));
    }
    auto *d = new fl_tensor_data_impl_t();
    d->ptr = p;
    d->numel = numel;
    d->dtype = dtype;
    d->device = device;
    d->owned = true;
    d->pooled = pooled;
    d->resident = resident;
    *out = d;
    return clear_error();
  });
}

int32_t fl_tensor_data_borrow(const void *data, fl_dtype_t dtype, int64_t numel, fl_tensor_data_t *out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    if (!data) invalid("data is null");
    if (numel < 1) invalid("storage holds at least one element");
    if (numel > kMaxStorageElements) invalid("too many elements");
    const int64_t alignment = dtype_size(dtype);
    if (reinterpret_cast<uintptr_t>(data) % alignment != 0) {
      invalid("data is not aligned to its " + std::to_string(alignment) + "-byte elements");
    }
    auto *d = new fl_tensor_data_impl_t();
    d->ptr = const_cast<void *>(data);
    d->numel = numel;
    d->dtype = dtype;
    d->device = FL_DEVICE_CPU;
    d->owned = false;
    *out = d;
    return clear_error();
  });
}

void fl_tensor_data_destroy(fl_tensor_data_t data) {
  if (!data) return;
  if (data->ipc_mapped && data->ptr) cudaIpcCloseMemHandle(data->ptr);
  if (data->owned && data->ptr) {
    switch (data->device) {
      case FL_DEVICE_CPU: free(data->ptr); break;
      case FL_DEVICE_CUDA:
        // In the order of the stream that last owned the bytes, so nothing waits; a weight's own
        // memory goes back with cudaFree, which waits for the device (flint/cuda/cuda_tensor_data.cc:62-77).
        if (data->pooled) {
          if (data->home && data->home != data->stream) {
            cudaEvent_t used = nullptr;
            if (cudaEventCreateWithFlags(&used, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventRecord(used, data->stream) == cudaSuccess) {
              std::lock_guard<std::mutex> lock(g_mutex);
              g_dev.returning.push_back({data->ptr, used, data->home});
              sweep_returning_locked(false);
            } else {
              if (used) cudaEventDestroy(used);
              cudaFreeAsync(data->ptr, data->stream);
            }
          } else {
            cudaFreeAsync(data->ptr, data->stream);
          }
        } else {
          cudaFree(data->ptr);
        }
        break;
      case FL_DEVICE_CUDA_HOST: cudaFreeHost(data->ptr); break;
      default: break;
    }
  }
  delete data;
}

int32_t fl_tensor_data_get_host_ptr(fl_tensor_data_t data, void **out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    fl_tensor_data_impl_t &d = deref(data);
    if (d.device != FL_DEVICE_CPU && d.device != FL_DEVICE_CUDA_HOST) {
      invalid(std::string("storage on ") + device_name(d.device) + " has no address the caller may touch");
    }
    *out = d.ptr;
    return clear_error();
  });
}

int32_t fl_tensor_view_create(fl_tensor_data_t data, const int32_t *shape, const int32_t *stride, int32_t ndim,
                              int64_t offset, fl_tensor_view_t *out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    fl_tensor_data_impl_t &storage = deref(data);
    if (ndim < 0) invalid("ndim must not be negative");
    if (ndim > 0 && (!shape || !stride)) invalid("shape or stride is null");
    if (offset < 0) invalid("offset must not be negative");
    int64_t last = offset;
    bool empty = false;
    for (int32_t d = 0; d < ndim; ++d) {
      if (shape[d] < 0) invalid("shape must not be negative");
      if (stride[d] < 0) invalid("stride must not be negative");
      if (shape[d] == 0) empty = true;
      last += static_cast<int64_t>(shape[d] > 0 ? shape[d] - 1 : 0) * stride[d];
    }
    if (!empty && last >= storage.numel) {
      invalid("the view reaches element " + std::to_string(last) + " of storage holding " +
              std::to_string(storage.numel));
    }
    auto *v = new fl_tensor_view_impl_t();
    v->data = &storage;
    v->shape.assign(shape, shape + ndim);
    v->stride.assign(stride, stride + ndim);
    v->offset = offset;
    *out = v;
    return clear_error();
  });
}

void fl_tensor_view_destroy(fl_tensor_view_t view) { delete view; }

int32_t fl_transfer(fl_operators_t operators, fl_tensor_view_t src_h, fl_tensor_view_t dest_h) {
  return guard([&]() {
    if (!operators) invalid("operators is null");
    fl_tensor_view_impl_t &src = deref(src_h);
    fl_tensor_view_impl_t &dest = deref(dest_h);
    if (!is_contiguous(src) || !is_contiguous(dest)) invalid("transfer: both views have to be contiguous");
    if (src.shape != dest.shape) invalid("transfer: the shapes differ");
    if (dtype_of(src) != dtype_of(dest)) invalid("transfer: the dtypes differ");
    const bool src_host = device_of(src) != FL_DEVICE_CUDA;
    const bool dest_host = device_of(dest) != FL_DEVICE_CUDA;
    if (src_host == dest_host) invalid("transfer: one side has to be on the device and the other on the host");
    check_earlier_kernel_status();
    const size_t bytes = static_cast<size_t>(numel_of(src) * dtype_size(dtype_of(src)));
    if (bytes == 0) return clear_error();
    cuda_check(cudaMemcpyAsync(raw_ptr(dest), raw_ptr(src), bytes,
                               src_host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, 0),
               "cudaMemcpyAsync");
    if (dest_host) {
      // The host is about to read the bytes: wait for them, and do not hand back the output of a
      // kernel that gave up on a wait, whichever status word it reported through.
      cuda_check(cudaStreamSynchronize(0), "cudaStreamSynchronize");
      check_earlier_kernel_status();
      const uint32_t code = take_static_status();
      if (code != 0) {
        aborted("a kernel of fl_fp8_linear_static gave up on a bounded wait (status " + std::to_string(code) + ")");
      }
    }
    return clear_error();
  });
}

// flint/capi.h:256-264, flint/cuda/to_device.cc:143-181. Page-locked host memory to the GPU, on
// the upload stream, into storage allocated in that stream's order; every other direction is
// refused rather than quietly done synchronously.
int32_t fl_transfer_async(fl_tensor_view_t src_h, fl_device_type_t device, fl_tensor_data_t *dest, fl_transfer_t *out) {
  return guard([&]() -> int32_t {
    if (!dest || !out) invalid("out is null");
    const fl_tensor_view_impl_t &src = deref(src_h);
    if (device != FL_DEVICE_CUDA || device_of(src) != FL_DEVICE_CUDA_HOST) {
      invalid(std::string("an asynchronous copy goes from cuda-host to cuda, not from ") + device_name(device_of(src)) +
              " to " + device_name(device));
    }
    if (!is_contiguous(src)) invalid("an asynchronous copy reads one contiguous run");
    require_kernels();
    ensure_pool();
    cudaStream_t stream = copy_stream(/*upload=*/true);
    const int64_t numel = numel_of(src);
    const size_t bytes = static_cast<size_t>(numel * dtype_size(dtype_of(src)));
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      sweep_returning_locked(false);
    }
    void *p = nullptr;
    cuda_check(cudaMallocAsync(&p, bytes ? bytes : 1, stream), "cudaMallocAsync");
    auto *d = new fl_tensor_data_impl_t();
    d->ptr = p;
    d->numel = numel > 0 ? numel : 1;
    d->dtype = dtype_of(src);
    d->device = FL_DEVICE_CUDA;
    d->owned = true;
    d->pooled = true;
    d->stream = stream;  // until the transfer is waited on, the copy stream owns the bytes
    d->home = stream;
    auto *t = new fl_transfer_impl_t();
    t->dest = d;
    cudaError_t e = bytes ? cudaMemcpyAsync(p, raw_ptr(src), bytes, cudaMemcpyHostToDevice, stream) : cudaSuccess;
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&t->event, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(t->event, stream);
    if (e != cudaSuccess) {
      if (t->event) cudaEventDestroy(t->event);
      delete t;
      fl_tensor_data_destroy(d);
      cuda_check(e, "starting the asynchronous copy");
    }
    *dest = d;
    *out = t;
    return clear_error();
  });
}

namespace {
// flint/cuda/to_device.cc:183-195: the compute stream waits rather than the host, unless the host
// is about to read the bytes itself; the storage then belongs to the compute stream.
int32_t wait_transfer(fl_transfer_t transfer, bool sync) {
  return guard([&]() -> int32_t {
    if (!transfer) invalid("transfer is null");
    if (transfer->event) {
      if (sync) {
        cuda_check(cudaEventSynchronize(transfer->event), "cudaEventSynchronize");
      } else {
        cuda_check(cudaStreamWaitEvent(0, transfer->event, 0), "cudaStreamWaitEvent");
      }
      if (transfer->dest) transfer->dest->stream = nullptr;
      cudaEventDestroy(transfer->event);
      transfer->event = nullptr;
    }
    return clear_error();
  });
}
}  // namespace

int32_t fl_transfer_wait(fl_transfer_t transfer) { return wait_transfer(transfer, false); }
int32_t fl_transfer_wait_sync(fl_transfer_t transfer) { return wait_transfer(transfer, true); }

void fl_transfer_destroy(fl_transfer_t transfer) {
  if (!transfer) return;
  if (transfer->event) cudaEventDestroy(transfer->event);  // a pending event goes once the device has reached it
  delete transfer;
}

// The other direction, which the reference only has synchronously (flint/cuda/to_device.cc:60-66):
// contiguous device `src` into page-locked host `dest`, on the download stream, ordered behind the
// work queued on the compute stream so far. fl_transfer_wait_sync() on the handle is when the host
// may read `dest`; `src` has to stay alive until then.
int32_t fl_sm100_transfer_to_host_async(fl_tensor_view_t src_h, fl_tensor_view_t dest_h, fl_transfer_t *out) {
  return guard([&]() -> int32_t {
    if (!out) invalid("out is null");
    const fl_tensor_view_impl_t &src = deref(src_h);
    const fl_tensor_view_impl_t &dest = deref(dest_h);
    if (device_of(src) != FL_DEVICE_CUDA || device_of(dest) != FL_DEVICE_CUDA_HOST) {
      invalid(std::string("an asynchronous download goes from cuda to cuda-host, not from ") + device_name(device_of(src)) +
              " to " + device_name(device_of(dest)));
    }
    if (!is_contiguous(src) || !is_contiguous(dest)) invalid("transfer: both views have to be contiguous");
    if (src.shape != dest.shape) invalid("transfer: the shapes differ");
    if (dtype_of(src) != dtype_of(dest)) invalid("transfer: the dtypes differ");
    require_kernels();
    check_earlier_kernel_status();
    cudaStream_t stream = copy_stream(/*upload=*/false);
    const size_t bytes = static_cast<size_t>(numel_of(src) * dtype_size(dtype_of(src)));
    auto *t = new fl_transfer_impl_t();
    cudaEvent_t produced = nullptr;
    cudaError_t e = cudaEventCreateWithFlags(&produced, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(produced, 0);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, produced, 0);
    if (produced) cudaEventDestroy(produced);
    if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(raw_ptr(dest), raw_ptr(src), bytes, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&t->event, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(t->event, stream);
    if (e != cudaSuccess) {
      if (t->event) cudaEventDestroy(t->event);
      delete t;
      cuda_check(e, "starting the asynchronous download");
    }
    *out = t;
    return clear_error();
  });
}

int32_t fl_fp8_available(fl_device_type_t device, int32_t *out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    if (device < FL_DEVICE_CPU || device > FL_DEVICE_UNKNOWN) invalid("unknown device");
    DeviceState &d = device_state();
    *out = (device == FL_DEVICE_CUDA && d.present && d.sm100) ? 1 : 0;
    return clear_error();
  });
}

int32_t fl_fp8_matmul(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scale, fl_tensor_view_t out) {
  return fl_fp8_matmul_add(a, data, scale, nullptr, out);
}

int32_t fl_fp8_matmul_add(fl_tensor_view_t a_h, fl_tensor_view_t data_h, fl_tensor_view_t scale_h,
                          fl_tensor_view_t addend_h, fl_tensor_view_t out_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &weight = deref(data_h);
    const fl_tensor_view_impl_t &scale = deref(scale_h);
    check_fp8_weight(weight, scale, /*per_channel_ok=*/false);
    const fl_device_type_t device = device_of(weight);
    const int rows = weight.shape[0];
    const int k = weight.shape[1];
    const fl_tensor_view_impl_t &a = deref(a_h);
    check_activation(a, device, "the left operand");
    if (a.shape.back() != k) invalid("the two operands disagree about k");
    const fl_tensor_view_impl_t &out = deref(out_h);
    check_result(out, a, rows, device);
    const fl_tensor_view_impl_t *addend = addend_h ? &deref(addend_h) : nullptr;
    if (addend) {
      if (device_of(*addend) != device || dtype_of(*addend) != dtype_of(out) ||
          addend->shape.size() > out.shape.size()) {
        invalid("the addend is not <float16> on the weight's device, of out's shape");
      }
    }
    if (device != FL_DEVICE_CUDA) invalid("the fp8 operand is on a device with no FP8 kernels");
    check_tiles(rows, k, 16);
    require_kernels();
    check_earlier_kernel_status();

    const int64_t m64 = leading_rows(a);
    if (m64 == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("the left operand has more rows than the kernels can index");
    const int m = static_cast<int>(m64);
    const int is_bf16 = dtype_of(a) == FL_DTYPE_BFLOAT16;

    // A handful of rows (the reference's decode shape): one bandwidth-shaped launch that widens
    // the weight in registers, with no scratch. An addend no epilogue can index goes the long way.
    {
      static const bool no_skinny = []() {
        const char *v = std::getenv("FLINT_SM100_NO_SKINNY");
        return v && v[0] == '1';
      }();
      AddendPlan quick;
      std::vector<int32_t> bs;
      std::vector<int64_t> bt;
      if (addend) quick = plan_addend(*addend, out, &bs, &bt);
      // Half rows against many channels: the weight on the M side of the tensor-core instruction
      // (fewrow_tc_sm100.cu). Its time, 5 us and 0.65 us per 256 K positions, depends neither on
      // the row count nor on the channel count up to 148 x 128 (a CTA per 128 channels, paced by
      // its own chain of stages), so it takes the products the kernel underneath is slower on, as
      // measured at 3072- and 12288-deep rows: any row count from 8192 channels, two rows or more
      // from 6144, eight or more from 3072; on shallower rows, where its fixed part weighs more,
      // only what was measured there. The instruction's time does not grow with its N, so 17 to 32
      // rows cost what 16 cost (32 x 16384 x 3072: 13.2 us against the tile kernel's 27.5) and 33
      // to 64 a little more (64 x 16384 x 3072: 14.9 us against 27.2).
      static const bool no_fewrow_tc = [] {
        const char *e = std::getenv("FLINT_SM100_NO_FEWROW_TC");
        return e && e[0] == '1';
      }();
      const bool fewrow_tc_wins = fewrow_tc_route(m, rows, k);
      if (!no_skinny && !no_fewrow_tc && !quick.needs_expand && fewrow_tc_wins &&
          fewrow_tc_supported(m, rows, k, is_bf16, raw_ptr(a), raw_ptr(weight), raw_ptr(out)) &&
          (!quick.residual || quick.residual_rows > 0)) {
        const char *why = "";
        cudaError_t e = fewrow_tc_matmul(raw_ptr(a), m, rows, k, reinterpret_cast<const uint8_t *>(raw_ptr(weight)),
                                         reinterpret_cast<const float *>(raw_ptr(scale)), quick.bias, quick.residual,
                                         quick.residual_rows, quick.residual_ld, raw_ptr(out), status_word(), 0, &why);
        if (e != cudaSuccess) cuda_check(e, (std::string("few-row FP8 matmul: ") + why).c_str());
        ++g_gemm_launches;
        return clear_error();
      }
      if (!no_skinny && !quick.needs_expand &&
          skinny_upcast_supported(m, rows, k, raw_ptr(a), raw_ptr(weight), raw_ptr(out), quick.residual != nullptr)) {
        cuda_check(skinny_upcast_matmul(raw_ptr(a), is_bf16, m, rows, k, raw_ptr(weight),
                                        reinterpret_cast<const float *>(raw_ptr(scale)), quick.bias, quick.residual,
                                        quick.residual_rows, quick.residual_ld, raw_ptr(out), status_word(), 0),
                   "skinny FP8 matmul");
        ++g_gemm_launches;
        return clear_error();
      }
    }

    // Half activations (the reference's contract): the 16-bit tcgen05 kernel in its mixed form. The
    // weight reaches shared memory as e4m3 bytes and is widened there, exactly, to half (flint widens
    // in registers inside its main loop, flint/cuda/gemm_fp8_cutlass.cu:142-149); the scale and the
    // addend go into the epilogue; no widened copy of the weight exists anywhere. Scratch is only
    // needed for operands whose view starts off a 16-byte boundary and for an addend no epilogue
    // can index.
    // bfloat16 activations (additive; the reference has none): one UMMA takes both operands in one
    // 16-bit format, and e4m3 -> bfloat16 has no conversion instruction, so the weight is widened
    // to bfloat16 by a pass of its own into scratch (rows * k * 2 bytes) and the plain kernel runs.
    Scratch scratch;
    size_t a_off = 0, w_off = 0;
    const bool a_misaligned = !aligned16(raw_ptr(a));
    const bool w_misaligned = !aligned16(raw_ptr(weight));
    if (a_misaligned) a_off = scratch.reserve(static_cast<size_t>(m) * k * 2);
    if (is_bf16) {
      w_off = scratch.reserve(static_cast<size_t>(rows) * k * 2);
    } else if (w_misaligned) {
      w_off = scratch.reserve(static_cast<size_t>(rows) * k);
    }
    AddendResolver res;
    res.prepare(addend, out, &scratch);
    uint8_t *base = scratch.used ? scratch.commit() : nullptr;

    const void *a_ptr = raw_ptr(a);
    const void *w_ptr = raw_ptr(weight);
    if (a_misaligned) {
      cuda_check(cudaMemcpyAsync(base + a_off, a_ptr, static_cast<size_t>(m) * k * 2, cudaMemcpyDeviceToDevice, 0),
                 "staging the left operand");
      a_ptr = base + a_off;
    }
    if (is_bf16) {
      cuda_check(widen_e4m3(raw_ptr(weight), static_cast<int64_t>(rows) * k, base + w_off, 1, 0), "widening");
      w_ptr = base + w_off;
    } else if (w_misaligned) {
      cuda_check(cudaMemcpyAsync(base + w_off, w_ptr, static_cast<size_t>(rows) * k, cudaMemcpyDeviceToDevice, 0),
                 "staging the weight");
      w_ptr = base + w_off;
    }
    Epilogue ep;
    ep.col_scale = reinterpret_cast<const float *>(raw_ptr(scale));
    ep.col_scale_scalar = 1;
    res.resolve(base, m, rows, &ep);
    run_gemm(is_bf16 ? kGemmBF16 : kGemmF16, m, rows, k, a_ptr, w_ptr, nullptr, nullptr, ep, is_bf16, raw_ptr(out),
             /*b_is_e4m3=*/!is_bf16);
    return clear_error();
  });
}

int32_t fl_matmul_add(fl_operators_t operators, fl_tensor_view_t a_h, fl_tensor_view_t b_h, fl_tensor_view_t addend_h,
                      fl_tensor_view_t out_h);

int32_t fl_matmul(fl_operators_t operators, fl_tensor_view_t a, fl_tensor_view_t b, fl_tensor_view_t out) {
  return fl_matmul_add(operators, a, b, nullptr, out);
}

// flint/capi.h:440-456, flint/cuda/matmul.cc:96-146,315-343. The linear-layer case on 16-bit
// operands -- `b` the transposed view of a weight stored (n, k) row-major, which is how an
// unquantised Linear hands its weight over (waifu/src/layers.rs:230-246), n and k multiples of 8 --
// runs on the tcgen05 tile kernel (at most 16 rows: the few-row kernel). Everything else the
// reference's matmul takes -- float32 operands, a float32 result from half operands, batches on
// either side, other layouts of `b`, odd extents -- runs on the general kernel of
// matmul_simt_sm100.cu.
int32_t fl_matmul_add(fl_operators_t operators, fl_tensor_view_t a_h, fl_tensor_view_t b_h, fl_tensor_view_t addend_h,
                      fl_tensor_view_t out_h) {
  return guard([&]() -> int32_t {
    if (!operators) invalid("operators is null");
    const fl_tensor_view_impl_t &a = deref(a_h);
    const fl_tensor_view_impl_t &b = deref(b_h);
    const fl_tensor_view_impl_t &out = deref(out_h);
    for (const fl_tensor_view_impl_t *v : {&a, &b, &out}) {
      if (device_of(*v) != FL_DEVICE_CUDA) invalid("an operand is not on the operators' device");
    }
    ElemKind in_kind, out_kind;
    if (!elem_kind_of(dtype_of(a), &in_kind) || dtype_of(b) != dtype_of(a) || !elem_kind_of(dtype_of(out), &out_kind) ||
        !(out_kind == in_kind || out_kind == kElemF32)) {
      invalid("matmul: operands of one type, <float>, <float16> or <bfloat16>, into a result of that type or <float>");
    }
    if (a.shape.size() < 2 || b.shape.size() < 2 || b.shape.size() > a.shape.size()) {
      invalid("matmul: both operands have at least two dimensions, the right one no more than the left");
    }
    const int ad = static_cast<int>(a.shape.size()), bd = static_cast<int>(b.shape.size());
    const int m_inner = a.shape[ad - 2], k = a.shape[ad - 1], n = b.shape[bd - 1];
    if (b.shape[bd - 2] != k) invalid("the two operands disagree about k");
    if (!is_contiguous(out)) invalid("out is not contiguous");
    std::vector<int32_t> shape = a.shape;
    shape.back() = n;
    check_shape(out, shape, "out");
    // the right operand's leading dimensions, aligned to the left one's from the right, equal or 1
    for (int i = 0; i < bd - 2; ++i) {
      const int32_t bs = b.shape[i], as = a.shape[ad - bd + i];
      if (bs != as && bs != 1) invalid("matmul: the right operand's leading dimensions do not broadcast over the left one's");
    }
    const fl_tensor_view_impl_t *addend = addend_h ? &deref(addend_h) : nullptr;
    if (addend) {
      if (device_of(*addend) != FL_DEVICE_CUDA || dtype_of(*addend) != dtype_of(out) ||
          addend->shape.size() > out.shape.size()) {
        invalid("matmul: the addend must be of the output's type and fit its shape");
      }
    }
    require_kernels();
    check_earlier_kernel_status();
    if (numel_of(out) == 0) return clear_error();
    const int64_t m64 = leading_rows(a);
    if (m64 > INT32_MAX) invalid("the left operand has more rows than the kernels can index");
    const int is_bf16 = dtype_of(a) == FL_DTYPE_BFLOAT16;

    // ---- the linear-layer case on 16-bit operands: tensor cores ----
    // (k, n) with strides (1, k): the transpose of a contiguous (n, k) weight.
    const bool k_major = bd == 2 && (b.stride[0] == 1 || k == 1) && (b.stride[1] == k || n == 1);
    if (in_kind != kElemF32 && out_kind == in_kind && k_major && is_contiguous(a) && n % 8 == 0 && k % 8 == 0 && k > 0) {
      const int m = static_cast<int>(m64);
      // A handful of rows (the reference keeps a GEMV for this, flint/cuda/matvec.cu): one
      // bandwidth-shaped launch with the bias or residual in its epilogue, no scratch.
      if (m <= 64) {
        static const bool no_skinny = []() {
          const char *v = std::getenv("FLINT_SM100_NO_SKINNY");
          return v && v[0] == '1';
        }();
        static const bool no_fewrow_tc = [] {
          const char *e = std::getenv("FLINT_SM100_NO_FEWROW_TC");
          return e && e[0] == '1';
        }();
        AddendPlan quick;
        std::vector<int32_t> bs;
        std::vector<int64_t> bt;
        if (addend) quick = plan_addend(*addend, out, &bs, &bt);
        // Against a wide weight: the weight on the M side of the tensor-core instruction
        // (fewrow_tc_sm100.cu), whose time does not grow with the rows.
        // Where it measured faster (1-64 rows, 3072-16384 channels, k = 3072 and 12288) than the
        // kernel underneath (at most 16 rows, mma.sync) and the tile kernel: 16 x 16384 x 3072
        // 19.3 us against 40.3, 32 x 8192 x 3072 15.0 against 21.9, 1 x 16384 x 12288 61.8 against
        // 77.9 (6.5 TB/s of weight).
        const bool fewrow_w16_wins = fewrow_w16_route(m, n, k);
        if (!no_skinny && !no_fewrow_tc && !quick.needs_expand && fewrow_w16_wins &&
            fewrow_w16_supported(m, n, k, raw_ptr(a), raw_ptr(b), raw_ptr(out)) && (!quick.residual || quick.residual_rows > 0)) {
          const char *why = "";
          cudaError_t e = fewrow_w16_matmul(raw_ptr(a), is_bf16, m, n, k, raw_ptr(b), quick.bias, quick.residual,
                                            quick.residual_rows, quick.residual_ld, raw_ptr(out), status_word(), 0, &why);
          if (e != cudaSuccess) cuda_check(e, (std::string("few-row matmul: ") + why).c_str());
          ++g_gemm_launches;
          return clear_error();
        }
        if (m <= 16 && !no_skinny && !quick.needs_expand &&
            skinny_w16_supported(m, n, k, raw_ptr(a), raw_ptr(b), raw_ptr(out), quick.residual != nullptr)) {
          cuda_check(skinny_w16_matmul(raw_ptr(a), is_bf16, m, n, k, raw_ptr(b), quick.bias, quick.residual, quick.residual_rows,
                                       quick.residual_ld, raw_ptr(out), status_word(), 0),
                     "few-row matmul");
          ++g_gemm_launches;
          return clear_error();
        }
      }
      Scratch scratch;
      size_t a_off = 0, b_off = 0;
      const bool a_misaligned = !aligned16(raw_ptr(a));
      const bool b_misaligned = !aligned16(raw_ptr(b));
      if (a_misaligned) a_off = scratch.reserve(static_cast<size_t>(m) * k * 2);
      if (b_misaligned) b_off = scratch.reserve(static_cast<size_t>(n) * k * 2);
      AddendResolver res;
      res.prepare(addend, out, &scratch);
      uint8_t *base = scratch.used ? scratch.commit() : nullptr;
      const void *a_ptr = raw_ptr(a);
      const void *b_ptr = raw_ptr(b);
      if (a_misaligned) {
        cuda_check(cudaMemcpyAsync(base + a_off, a_ptr, static_cast<size_t>(m) * k * 2, cudaMemcpyDeviceToDevice, 0), "staging");
        a_ptr = base + a_off;
      }
      if (b_misaligned) {
        cuda_check(cudaMemcpyAsync(base + b_off, b_ptr, static_cast<size_t>(n) * k * 2, cudaMemcpyDeviceToDevice, 0), "staging");
        b_ptr = base + b_off;
      }
      Epilogue ep;
      res.resolve(base, m, n, &ep);
      run_gemm(is_bf16 ? kGemmBF16 : kGemmF16, m, n, k, a_ptr, b_ptr, nullptr, nullptr, ep, is_bf16, raw_ptr(out));
      return clear_error();
    }

    // ---- every other case: the general kernel ----
    GeneralMatmulArgs g = {};
    g.a = raw_ptr(a);
    g.b = raw_ptr(b);
    g.out = raw_ptr(out);
    g.in_kind = in_kind;
    g.out_kind = out_kind;
    g.n = n;
    g.k = k;
    g.a_col = a.stride[ad - 1];
    g.b_row = b.stride[bd - 2];
    g.b_col = b.stride[bd - 1];
    g.stream = 0;
    if (bd == 2 && is_contiguous(a)) {
      // one right operand for every row of a contiguous left one: the leading dimensions fold into m
      g.m = static_cast<int>(m64);
      g.a_row = k;
      g.a_col = 1;
      g.batch_dims = 0;
    } else {
      g.m = m_inner;
      g.a_row = a.stride[ad - 2];
      const int lead = ad - 2;
      if (lead > kMaxMatmulBatchDims) {
        invalid("matmul: more than " + std::to_string(kMaxMatmulBatchDims) + " leading dimensions on a batched product");
      }
      g.batch_dims = lead;
      int64_t batches = 1;
      for (int i = 0; i < lead; ++i) {
        g.batch_shape[i] = a.shape[i];
        g.a_batch[i] = a.shape[i] == 1 ? 0 : a.stride[i];
        const int bi = i - (ad - bd);  // the right operand's dimension under this one, if it has it
        g.b_batch[i] = (bi >= 0 && b.shape[bi] != 1) ? b.stride[bi] : 0;
        batches *= a.shape[i];
      }
      if (batches > 65535) invalid("matmul: more than 65535 products in a batch");
    }
    Scratch scratch;
    AddendResolver res;
    res.prepare(addend, out, &scratch);
    uint8_t *base = nullptr;
    if (scratch.used) {
      if (out_kind == kElemF32 && res.plan.needs_expand) {
        invalid("matmul: a <float> addend has to be a bias or a residual laid out as rows of out");
      }
      base = scratch.commit();
    }
    Epilogue ep;
    res.resolve(base, static_cast<int>(m64), n, &ep);
    g.bias = ep.bias;
    g.residual = ep.residual;
    g.residual_rows = ep.residual_rows;
    g.residual_ld = ep.residual_ld;
    cuda_check(general_matmul(g), "matmul");
    return clear_error();
  });
}

// ---- the elementwise operators around the path (flint/capi.h:246-249,279,483) -------------------

namespace {

ElemView elem_view(const fl_tensor_view_impl_t &v, const char *what) {
  if (v.shape.size() > static_cast<size_t>(kMaxElemDims)) {
    invalid(std::string(what) + " has more than " + std::to_string(kMaxElemDims) + " dimensions");
  }
  ElemView e = {};
  e.base = raw_ptr(v);
  e.ndim = static_cast<int>(v.shape.size());
  for (int d = 0; d < e.ndim; ++d) {
    e.shape[d] = v.shape[d];
    e.stride[d] = v.stride[d];
  }
  e.contiguous = is_contiguous(v);
  return e;
}

// flint/capi.cc:176-189 (checkOnDevice): every view of an operation is on the operators' device.
void check_on_cuda(fl_operators_t operators, const fl_tensor_view_impl_t &v, const char *what) {
  if (!operators) invalid("operators is null");
  if (device_of(v) != FL_DEVICE_CUDA) invalid(std::string(what) + " is not on the operators' device");
}

}  // namespace

// flint/capi.h:246, flint/capi.cc:478-501. Same shape and dtype; any strides.
int32_t fl_copy(fl_operators_t operators, fl_tensor_view_t src_h, fl_tensor_view_t dest_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &src = deref(src_h);
    const fl_tensor_view_impl_t &dest = deref(dest_h);
    check_on_cuda(operators, src, "the source");
    check_on_cuda(operators, dest, "the destination");
    if (dtype_of(src) != dtype_of(dest)) invalid("the source and the destination hold different types");
    check_shape(dest, src.shape, "the destination");
    require_kernels();
    cuda_check(elementwise_copy(elem_view(src, "the source"), elem_view(dest, "the destination"),
                                static_cast<int>(dtype_size(dtype_of(src))), numel_of(src), 0),
               "copy");
    return clear_error();
  });
}

// flint/capi.h:249, flint/capi.cc:503-507. Between <float>, <float16> and <bfloat16>, any strides
// (the reference's CUDA cast serves float <-> float16 on contiguous views, flint/cuda/cast.cu:70-95).
int32_t fl_cast(fl_operators_t operators, fl_tensor_view_t input_h, fl_tensor_view_t out_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &x = deref(input_h);
    const fl_tensor_view_impl_t &y = deref(out_h);
    check_on_cuda(operators, x, "the input");
    check_on_cuda(operators, y, "out");
    check_shape(y, x.shape, "out");
    ElemKind from, to;
    if (!elem_kind_of(dtype_of(x), &from) || !elem_kind_of(dtype_of(y), &to)) {
      invalid("cast: this library converts between <float>, <float16> and <bfloat16>");
    }
    require_kernels();
    cuda_check(elementwise_cast(elem_view(x, "the input"), from, elem_view(y, "out"), to, numel_of(x), 0), "cast");
    return clear_error();
  });
}

// flint/capi.h:279, flint/capi.cc:620-624.
int32_t fl_fill(fl_operators_t operators, fl_tensor_view_t tensor_h, float value) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &t = deref(tensor_h);
    check_on_cuda(operators, t, "the tensor");
    ElemKind kind;
    if (!elem_kind_of(dtype_of(t), &kind)) invalid("fill: this library fills <float>, <float16> and <bfloat16> tensors");
    require_kernels();
    cuda_check(elementwise_fill(elem_view(t, "the tensor"), kind, numel_of(t), value, 0), "fill");
    return clear_error();
  });
}

// flint/capi.h:480-483, flint/capi.cc:226-252. `b` and `out` have `a`'s shape (a caller broadcasting
// a smaller operand hands over an expanded view of it); one dtype.
int32_t fl_add(fl_operators_t operators, fl_tensor_view_t a_h, fl_tensor_view_t b_h, fl_tensor_view_t out_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &a = deref(a_h);
    const fl_tensor_view_impl_t &b = deref(b_h);
    const fl_tensor_view_impl_t &out = deref(out_h);
    check_on_cuda(operators, a, "the left operand");
    check_on_cuda(operators, b, "the right operand");
    check_on_cuda(operators, out, "out");
    check_shape(b, a.shape, "the right operand");
    check_shape(out, a.shape, "out");
    ElemKind kind;
    if (!elem_kind_of(dtype_of(a), &kind) || dtype_of(b) != dtype_of(a) || dtype_of(out) != dtype_of(a)) {
      invalid("add: this library adds <float>, <float16> or <bfloat16> operands of one type");
    }
    require_kernels();
    cuda_check(elementwise_add(elem_view(a, "the left operand"), elem_view(b, "the right operand"), elem_view(out, "out"),
                               kind, numel_of(a), 0),
               "add");
    return clear_error();
  });
}

// ============================ Part 2 ==========================================================

namespace {
// At most 32 quantised rows against a wide weight: the weight on the M side of the tensor-core
// instruction (fewrow_tc_sm100.cu, fewrow_q8_kernel), where the tile kernel would stream it through
// the few SMs its tiles land on. `fewrow_q8_wins` is where it measured faster, quantiser launch
// included, than the tile kernel and (at most four rows) the one-launch kernel of skinny_sm100.cu,
// over 1-128 rows, 3072-18432 channels, k = 3072 and 12288: e.g. 16 x 16384 x 3072 14.5 us against
// 20.5, 1 x 16384 x 12288 35.4 against 63.0 (5.7 TB/s of weight); from 64 rows on the tile kernel
// is level or ahead.
bool fewrow_q8_wins(int m, int rows, int k) {
  static const bool off = [] {
    const char *a = std::getenv("FLINT_SM100_NO_SKINNY"), *b = std::getenv("FLINT_SM100_NO_FEWROW_TC");
    return (a && a[0] == '1') || (b && b[0] == '1');
  }();
  return !off && fewrow_q8_route(m, rows, k);
}

// Runs it if it wins and can take the operands; false when the tile kernel should run.
bool try_fewrow_q8(const uint8_t *codes, const float *row_scales, int m, int rows, int k, const void *w,
                   const Epilogue &ep, int is_bf16, void *out, uint32_t *status) {
  if (ep.row_amax != nullptr || ep.num_extra_out != 0 || ep.out_ld != 0) return false;
  if (!fewrow_q8_wins(m, rows, k) || !fewrow_q8_supported(m, rows, k, codes, w, out)) return false;
  const char *why = "";
  cudaError_t e = fewrow_q8_linear(codes, row_scales, m, rows, k, reinterpret_cast<const uint8_t *>(w), ep.col_scale,
                                   ep.col_scale_scalar, ep.bias, ep.residual, ep.residual_rows, ep.residual_ld, ep.act,
                                   is_bf16, out, status, 0, &why);
  if (e != cudaSuccess) cuda_check(e, (std::string("few-row FP8 linear: ") + why).c_str());
  ++g_gemm_launches;
  return true;
}

int32_t fp8_linear_impl(fl_tensor_view_t a_h, fl_tensor_view_t data_h, fl_tensor_view_t scales_h,
                        fl_tensor_view_t bias_h, fl_tensor_view_t residual_h, int32_t act, fl_tensor_view_t out_h,
                        fl_tensor_view_t row_amax_h, bool want_amax) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &weight = deref(data_h);
    const fl_tensor_view_impl_t &scales = deref(scales_h);
    check_fp8_weight(weight, scales, /*per_channel_ok=*/true);
    const fl_device_type_t device = device_of(weight);
    const int rows = weight.shape[0];
    const int k = weight.shape[1];
    const fl_tensor_view_impl_t &a = deref(a_h);
    check_activation(a, device, "the left operand");
    if (a.shape.back() != k) invalid("the two operands disagree about k");
    const fl_tensor_view_impl_t &out = deref(out_h);
    check_result(out, a, rows, device);
    if (act != FL_ACT_NONE && act != FL_ACT_GELU_TANH) invalid("unknown activation");
    const fl_tensor_view_impl_t *bias = bias_h ? &deref(bias_h) : nullptr;
    const fl_tensor_view_impl_t *residual = residual_h ? &deref(residual_h) : nullptr;
    if (bias) {
      if (device_of(*bias) != device || dtype_of(*bias) != dtype_of(out) || numel_of(*bias) != rows ||
          !is_contiguous(*bias)) {
        invalid("the bias is not a contiguous (rows) vector of out's type on the weight's device");
      }
    }
    if (residual) {
      if (device_of(*residual) != device || dtype_of(*residual) != dtype_of(out) || !is_contiguous(*residual)) {
        invalid("the residual is not contiguous, of out's type, on the weight's device");
      }
      check_shape(*residual, out.shape, "the residual");
    }
    if (device != FL_DEVICE_CUDA) invalid("the fp8 operand is on a device with no FP8 kernels");
    check_tiles(rows, k, 16);
    require_kernels();
    check_earlier_kernel_status();

    const int64_t m64 = leading_rows(a);
    if (m64 == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("the left operand has more rows than the kernels can index");
    const int m = static_cast<int>(m64);
    const int is_bf16 = dtype_of(a) == FL_DTYPE_BFLOAT16;

    // One to four rows: one bandwidth-shaped launch that quantises, streams the weight once and
    // applies the epilogue, with no scratch at all. From five rows on, every CTA quantising all
    // the rows for itself costs more than the separate quantiser launch of the tile path saves.
    static const bool no_skinny = []() {
      const char *v = std::getenv("FLINT_SM100_NO_SKINNY");
      return v && v[0] == '1';
    }();
    float *row_amax = nullptr;
    if (want_amax) {
      const fl_tensor_view_impl_t &am = deref(row_amax_h);
      if (dtype_of(am) != FL_DTYPE_FLOAT || numel_of(am) != m64 || !is_contiguous(am) || device_of(am) != device) {
        invalid("row_amax is not a contiguous <float> tensor of one value per row on the weight's device");
      }
      row_amax = reinterpret_cast<float *>(raw_ptr(am));
      cuda_check(cudaMemsetAsync(row_amax, 0, static_cast<size_t>(m) * sizeof(float), 0), "clearing the row maxima");
    }
    if (!want_amax && !no_skinny && m <= 4 && !(aligned16(raw_ptr(weight)) && fewrow_q8_wins(m, rows, k)) &&
        skinny_fp8_supported(m, rows, k, raw_ptr(a), raw_ptr(weight), raw_ptr(out), residual != nullptr)) {
      cuda_check(skinny_fp8_linear(raw_ptr(a), is_bf16, m, rows, k, raw_ptr(weight),
                                   reinterpret_cast<const float *>(raw_ptr(scales)), numel_of(scales) == 1 ? 1 : 0,
                                   bias ? raw_ptr(*bias) : nullptr, residual ? raw_ptr(*residual) : nullptr, act,
                                   raw_ptr(out), status_word(), 0),
                 "skinny FP8 linear");
      ++g_gemm_launches;
      return clear_error();
    }

    Scratch scratch;
    const size_t codes_off = scratch.reserve(static_cast<size_t>(m) * k);
    const size_t scales_off = scratch.reserve(static_cast<size_t>(m) * 4);
    size_t w_off = 0;
    const bool w_misaligned = !aligned16(raw_ptr(weight));
    if (w_misaligned) w_off = scratch.reserve(static_cast<size_t>(rows) * k);
    uint8_t *base = scratch.commit();

    uint8_t *codes = base + codes_off;
    float *row_scales = reinterpret_cast<float *>(base + scales_off);
    cuda_check(quantize_fp8_act(raw_ptr(a), is_bf16, m, k, codes, row_scales, 0), "quantising the activation");
    const void *w_ptr = raw_ptr(weight);
    if (w_misaligned) {
      cuda_check(cudaMemcpyAsync(base + w_off, w_ptr, static_cast<size_t>(rows) * k, cudaMemcpyDeviceToDevice, 0),
                 "staging the weight");
      w_ptr = base + w_off;
    }
    Epilogue ep;
    ep.row_scale = row_scales;
    ep.col_scale = reinterpret_cast<const float *>(raw_ptr(scales));
    ep.col_scale_scalar = numel_of(scales) == 1 ? 1 : 0;
    ep.bias = bias ? raw_ptr(*bias) : nullptr;
    if (residual) {
      ep.residual = raw_ptr(*residual);
      ep.residual_rows = m;
      ep.residual_ld = rows;
    }
    ep.act = act;
    ep.row_amax = row_amax;
    if (try_fewrow_q8(codes, row_scales, m, rows, k, w_ptr, ep, is_bf16, raw_ptr(out), status_word())) return clear_error();
    run_gemm(kGemmE4M3, m, rows, k, codes, w_ptr, nullptr, nullptr, ep, is_bf16, raw_ptr(out));
    return clear_error();
  });
}
}  // namespace

int32_t fl_fp8_linear(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scales, fl_tensor_view_t bias,
                      fl_tensor_view_t residual, int32_t act, fl_tensor_view_t out) {
  return fp8_linear_impl(a, data, scales, bias, residual, act, out, nullptr, false);
}

int32_t fl_fp8_linear_amax(fl_tensor_view_t a, fl_tensor_view_t data, fl_tensor_view_t scales, fl_tensor_view_t bias,
                           fl_tensor_view_t residual, int32_t act, fl_tensor_view_t out, fl_tensor_view_t row_amax) {
  return fp8_linear_impl(a, data, scales, bias, residual, act, out, row_amax, true);
}

// The second half of a narrow gather: this rank's column block of a 16-bit matrix, quantised per
// row with the rows' maxima over the whole matrix (fl_fp8_linear_amax's output after a maximum
// over the ranks), written as e4m3 codes into the same columns of every rank's full-width matrix.
int32_t fl_fp8_quantize_scatter(fl_tensor_view_t x_h, fl_tensor_view_t row_amax_h, const fl_tensor_view_t *dests,
                                int32_t n_dest, int32_t col0, fl_tensor_view_t row_scales_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &x = deref(x_h);
    const fl_tensor_view_impl_t &am = deref(row_amax_h);
    if (!is_half_type(dtype_of(x)) || x.shape.size() < 2 || !is_contiguous(x) || device_of(x) != FL_DEVICE_CUDA) {
      invalid("x is not a contiguous <float16> or <bfloat16> tensor of at least two dimensions on cuda");
    }
    const int64_t m64 = leading_rows(x);
    const int k = x.shape.back();
    if (dtype_of(am) != FL_DTYPE_FLOAT || numel_of(am) != m64 || !is_contiguous(am) || device_of(am) != FL_DEVICE_CUDA) {
      invalid("row_amax is not a contiguous <float> tensor of one value per row of x on cuda");
    }
    if (!dests || n_dest < 1 || n_dest > kMaxGemmOutputs) {
      invalid("scatter: between 1 and " + std::to_string(kMaxGemmOutputs) + " destinations are needed");
    }
    const fl_tensor_view_impl_t &first = deref(dests[0]);
    if (first.shape.size() != x.shape.size()) invalid("scatter: a destination has not x's rank");
    const int64_t ld = first.shape.back();
    if (col0 < 0 || col0 + static_cast<int64_t>(k) > ld) invalid("scatter: the column block does not fit the destination");
    if (k % 16 != 0 || ld % 16 != 0 || col0 % 16 != 0) invalid("scatter: x's width, the destination's width and the column offset are multiples of 16");
    uint8_t *ptrs[kMaxGemmOutputs];
    for (int i = 0; i < n_dest; ++i) {
      const fl_tensor_view_impl_t &d = deref(dests[i]);
      if (device_of(d) != FL_DEVICE_CUDA || dtype_of(d) != FL_DTYPE_FP8E4M3 || !is_contiguous(d) || d.shape != first.shape) {
        invalid("scatter: the destinations are not contiguous <fp8e4m3> matrices of one shape on cuda");
      }
      for (size_t j = 0; j + 1 < x.shape.size(); ++j) {
        if (d.shape[j] != x.shape[j]) invalid("scatter: a destination has not x's leading dimensions");
      }
      if (!aligned16(raw_ptr(d))) invalid("scatter: a destination's first element is not 16-byte aligned");
      ptrs[i] = raw_ptr(d);
    }
    if (!aligned16(raw_ptr(x))) invalid("scatter: x's first element is not 16-byte aligned");
    float *scales_out = nullptr;
    if (row_scales_h) {
      const fl_tensor_view_impl_t &rs = deref(row_scales_h);
      if (dtype_of(rs) != FL_DTYPE_FLOAT || numel_of(rs) != m64 || !is_contiguous(rs) || device_of(rs) != FL_DEVICE_CUDA) {
        invalid("row_scales is not a contiguous <float> tensor of one value per row of x on cuda");
      }
      scales_out = reinterpret_cast<float *>(raw_ptr(rs));
    }
    require_kernels();
    check_earlier_kernel_status();
    if (m64 == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("x has more rows than the kernel can index");
    cuda_check(quantize_fp8_scatter(raw_ptr(x), dtype_of(x) == FL_DTYPE_BFLOAT16, static_cast<int>(m64), k,
                                    reinterpret_cast<const float *>(raw_ptr(am)), ptrs, n_dest, ld, col0, scales_out, 0),
               "quantising and scattering");
    return clear_error();
  });
}

namespace {

// The destinations of a scattering epilogue: contiguous (..., ld) matrices of one shape with the left
// operand's leading dimensions, of the product's type, on the device; the product lands in columns
// [col0, col0 + rows) of each.
struct ScatterDests {
  void *first = nullptr;
  void *extra[kMaxGemmOutputs] = {};
  int num_extra = 0;
  int64_t ld = 0;
};

ScatterDests check_scatter_dests(const fl_tensor_view_t *dests, int32_t n_dest, int32_t col0, int rows,
                                 const std::vector<int32_t> &left_shape, fl_dtype_t dtype, fl_device_type_t device) {
  if (!dests || n_dest < 1 || n_dest > kMaxGemmOutputs) {
    invalid("scatter: between 1 and " + std::to_string(kMaxGemmOutputs) + " destinations are needed");
  }
  const fl_tensor_view_impl_t &first = deref(dests[0]);
  if (first.shape.size() != left_shape.size()) invalid("scatter: a destination has not the left operand's rank");
  ScatterDests out;
  out.ld = first.shape.back();
  if (col0 < 0 || col0 + static_cast<int64_t>(rows) > out.ld) invalid("scatter: the column block does not fit the destination");
  if (out.ld % 8 != 0 || col0 % 8 != 0) invalid("scatter: the destination's width and the column offset are multiples of 8");
  for (int i = 0; i < n_dest; ++i) {
    const fl_tensor_view_impl_t &d = deref(dests[i]);
    if (device_of(d) != device || dtype_of(d) != dtype || !is_contiguous(d) || d.shape != first.shape) {
      invalid("scatter: the destinations are not contiguous matrices of one shape, of the product's type, on the device");
    }
    for (size_t j = 0; j + 1 < left_shape.size(); ++j) {
      if (d.shape[j] != left_shape[j]) invalid("scatter: a destination has not the left operand's leading dimensions");
    }
    if (!aligned16(raw_ptr(d))) invalid("scatter: a destination's first element is not 16-byte aligned");
    if (i == 0) out.first = raw_ptr(d);
    else out.extra[out.num_extra++] = raw_ptr(d);
  }
  return out;
}

}  // namespace

int32_t fl_fp8_row_amax(fl_tensor_view_t x_h, fl_tensor_view_t row_amax_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &x = deref(x_h);
    const fl_tensor_view_impl_t &am = deref(row_amax_h);
    if (!is_half_type(dtype_of(x)) || x.shape.size() != 2 || x.stride[1] != 1 || device_of(x) != FL_DEVICE_CUDA) {
      invalid("x is not a <float16> or <bfloat16> matrix with contiguous rows on cuda");
    }
    if (dtype_of(am) != FL_DTYPE_FLOAT || numel_of(am) != x.shape[0] || !is_contiguous(am) || device_of(am) != FL_DEVICE_CUDA) {
      invalid("row_amax is not a contiguous <float> tensor of one value per row of x on cuda");
    }
    require_kernels();
    check_earlier_kernel_status();
    if (x.shape[0] == 0) return clear_error();
    cuda_check(row_amax_16(raw_ptr(x), dtype_of(x) == FL_DTYPE_BFLOAT16, x.shape[0], x.shape[1], x.stride[0],
                           reinterpret_cast<float *>(raw_ptr(am)), 0),
               "taking the rows' maxima");
    return clear_error();
  });
}

int32_t fl_fp8_linear_scatter(fl_tensor_view_t a_h, fl_tensor_view_t data_h, fl_tensor_view_t scales_h,
                              fl_tensor_view_t bias_h, fl_tensor_view_t residual_h, int32_t act,
                              const fl_tensor_view_t *dests, int32_t n_dest, int32_t col0) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &weight = deref(data_h);
    const fl_tensor_view_impl_t &scales = deref(scales_h);
    check_fp8_weight(weight, scales, /*per_channel_ok=*/true);
    const fl_device_type_t device = device_of(weight);
    const int rows = weight.shape[0];
    const int k = weight.shape[1];
    const fl_tensor_view_impl_t &a = deref(a_h);
    check_activation(a, device, "the left operand");
    if (a.shape.back() != k) invalid("the two operands disagree about k");
    if (act != FL_ACT_NONE && act != FL_ACT_GELU_TANH) invalid("unknown activation");
    const ScatterDests sd = check_scatter_dests(dests, n_dest, col0, rows, a.shape, dtype_of(a), device);
    const fl_tensor_view_impl_t *bias = bias_h ? &deref(bias_h) : nullptr;
    const fl_tensor_view_impl_t *residual = residual_h ? &deref(residual_h) : nullptr;
    if (bias) {
      if (device_of(*bias) != device || dtype_of(*bias) != dtype_of(a) || numel_of(*bias) != rows || !is_contiguous(*bias)) {
        invalid("the bias is not a contiguous (rows) vector of the product's type on the weight's device");
      }
    }
    if (residual) {
      std::vector<int32_t> shape = a.shape;
      shape.back() = rows;
      if (device_of(*residual) != device || dtype_of(*residual) != dtype_of(a) || !is_contiguous(*residual)) {
        invalid("the residual is not contiguous, of the product's type, on the weight's device");
      }
      check_shape(*residual, shape, "the residual");
    }
    if (device != FL_DEVICE_CUDA) invalid("the fp8 operand is on a device with no FP8 kernels");
    check_tiles(rows, k, 16);
    require_kernels();
    check_earlier_kernel_status();

    const int64_t m64 = leading_rows(a);
    if (m64 == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("the left operand has more rows than the kernels can index");
    const int m = static_cast<int>(m64);
    const int is_bf16 = dtype_of(a) == FL_DTYPE_BFLOAT16;

    Scratch scratch;
    const size_t codes_off = scratch.reserve(static_cast<size_t>(m) * k);
    const size_t scales_off = scratch.reserve(static_cast<size_t>(m) * 4);
    size_t w_off = 0;
    const bool w_misaligned = !aligned16(raw_ptr(weight));
    if (w_misaligned) w_off = scratch.reserve(static_cast<size_t>(rows) * k);
    uint8_t *base = scratch.commit();
    uint8_t *codes = base + codes_off;
    float *row_scales = reinterpret_cast<float *>(base + scales_off);
    cuda_check(quantize_fp8_act(raw_ptr(a), is_bf16, m, k, codes, row_scales, 0), "quantising the activation");
    const void *w_ptr = raw_ptr(weight);
    if (w_misaligned) {
      cuda_check(cudaMemcpyAsync(base + w_off, w_ptr, static_cast<size_t>(rows) * k, cudaMemcpyDeviceToDevice, 0),
                 "staging the weight");
      w_ptr = base + w_off;
    }
    Epilogue ep;
    ep.row_scale = row_scales;
    ep.col_scale = reinterpret_cast<const float *>(raw_ptr(scales));
    ep.col_scale_scalar = numel_of(scales) == 1 ? 1 : 0;
    ep.bias = bias ? raw_ptr(*bias) : nullptr;
    if (residual) {
      ep.residual = raw_ptr(*residual);
      ep.residual_rows = m;
      ep.residual_ld = rows;
    }
    ep.act = act;
    ep.out_ld = sd.ld;
    ep.out_col0 = col0;
    for (int i = 0; i < sd.num_extra; ++i) ep.extra_out[ep.num_extra_out++] = sd.extra[i];
    run_gemm(kGemmE4M3, m, rows, k, codes, w_ptr, nullptr, nullptr, ep, is_bf16, sd.first);
    return clear_error();
  });
}

int32_t fl_sm100_peer_exchange(const fl_tensor_view_t *mailboxes, int32_t n_ranks, int32_t rank, int32_t epoch,
                               fl_tensor_view_t row_amax_h, int32_t max_polls) {
  return guard([&]() -> int32_t {
    if (!mailboxes || n_ranks < 1 || n_ranks > kPeerMaxRanks) invalid("between 1 and " + std::to_string(kPeerMaxRanks) + " mailboxes are needed");
    if (rank < 0 || rank >= n_ranks) invalid("rank is not one of the mailboxes");
    if (epoch < 1) invalid("epochs start at 1 and grow");
    if (max_polls < 0) invalid("max_polls is not negative (0: the default limit)");
    PeerExchangeArgs args{};
    const fl_tensor_view_impl_t &first = deref(mailboxes[0]);
    if (first.shape.size() != 2 || first.shape[0] < n_ranks || first.shape[1] < kPeerHeaderWords) {
      invalid("a mailbox is an <int32>(n_ranks or more, " + std::to_string(kPeerHeaderWords) + " + rows) matrix");
    }
    for (int i = 0; i < n_ranks; ++i) {
      const fl_tensor_view_impl_t &b = deref(mailboxes[i]);
      if (dtype_of(b) != FL_DTYPE_INT32 || device_of(b) != FL_DEVICE_CUDA || !is_contiguous(b) || b.shape != first.shape) {
        invalid("the mailboxes are not contiguous <int32> matrices of one shape on cuda");
      }
      if (!aligned16(raw_ptr(b))) invalid("a mailbox's first element is not 16-byte aligned");
      args.mailbox[i] = reinterpret_cast<int32_t *>(raw_ptr(b));
    }
    args.n_ranks = n_ranks;
    args.rank = rank;
    args.ld = first.shape[1];
    args.epoch = epoch;
    if (row_amax_h) {
      const fl_tensor_view_impl_t &am = deref(row_amax_h);
      if (dtype_of(am) != FL_DTYPE_FLOAT || device_of(am) != FL_DEVICE_CUDA || !is_contiguous(am)) {
        invalid("row_amax is not a contiguous <float> tensor on cuda");
      }
      if (numel_of(am) > first.shape[1] - kPeerHeaderWords) invalid("row_amax has more values than a mailbox row holds");
      args.row_amax = reinterpret_cast<float *>(raw_ptr(am));
      args.rows = static_cast<int>(numel_of(am));
    }
    args.max_polls = static_cast<uint32_t>(max_polls);
    require_kernels();
    check_earlier_kernel_status();
    args.status = status_word();
    args.stream = 0;
    cuda_check(peer_exchange(args), "launching the peer exchange");
    ++g_block_launches;
    return clear_error();
  });
}

int32_t fl_sm100_ipc_export(fl_tensor_data_t data, void *handle_out) {
  return guard([&]() -> int32_t {
    fl_tensor_data_impl_t &d = deref(data);
    if (!handle_out) invalid("handle_out is null");
    if (d.device != FL_DEVICE_CUDA || !d.owned || !d.resident) {
      invalid("only device storage made by fl_tensor_data_create with FL_ALLOC_WEIGHT, of 2 MiB or more, can be exported "
              "(memory of the stream-ordered pool has no inter-process handle)");
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is documented as 64 bytes");
    cudaIpcMemHandle_t h;
    cuda_check(cudaIpcGetMemHandle(&h, d.ptr), "cudaIpcGetMemHandle");
    std::memcpy(handle_out, &h, sizeof(h));
    return clear_error();
  });
}

int32_t fl_sm100_ipc_import(const void *handle, fl_dtype_t dtype, int64_t numel, fl_tensor_data_t *out) {
  return guard([&]() -> int32_t {
    if (!handle) invalid("handle is null");
    if (!out) invalid("out is null");
    if (numel < 1) invalid("storage holds at least one element");
    dtype_size(dtype);
    require_kernels();
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void *ptr = nullptr;
    cuda_check(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    auto *d = new fl_tensor_data_impl_t();
    d->ptr = ptr;
    d->numel = numel;
    d->dtype = dtype;
    d->device = FL_DEVICE_CUDA;
    d->owned = false;
    d->ipc_mapped = true;
    *out = d;
    return clear_error();
  });
}

int32_t fl_nvfp4_available(fl_device_type_t device, int32_t *out) { return fl_fp8_available(device, out); }

int32_t fl_nvfp4_linear(fl_tensor_view_t a_h, fl_tensor_view_t codes_h, fl_tensor_view_t block_scales_h,
                        fl_tensor_view_t global_scale_h, fl_tensor_view_t bias_h, fl_tensor_view_t residual_h,
                        int32_t act, fl_tensor_view_t out_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &wcodes = deref(codes_h);
    const fl_tensor_view_impl_t &wsf = deref(block_scales_h);
    const fl_tensor_view_impl_t &gs = deref(global_scale_h);
    if (dtype_of(wcodes) != FL_DTYPE_FP4E2M1X2 || wcodes.shape.size() != 2) {
      invalid("nvfp4 operand: codes is not <fp4e2m1x2>(rows, k/2)");
    }
    const fl_device_type_t device = device_of(wcodes);
    const int rows = wcodes.shape[0];
    const int64_t k64 = static_cast<int64_t>(wcodes.shape[1]) * 2;
    if (k64 > INT32_MAX) invalid("nvfp4 operand: k is too large");
    const int k = static_cast<int>(k64);
    if (dtype_of(wsf) != FL_DTYPE_FP8E4M3 || wsf.shape.size() != 2 || wsf.shape[0] != rows ||
        static_cast<int64_t>(wsf.shape[1]) * 16 != k) {
      invalid("nvfp4 operand: block_scales is not <fp8e4m3>(rows, k/16)");
    }
    if (dtype_of(gs) != FL_DTYPE_FLOAT || numel_of(gs) != 1) invalid("nvfp4 operand: the global scale is not a single <float>");
    if (device_of(wsf) != device || device_of(gs) != device) invalid("nvfp4 operand: its parts are on different devices");
    if (!is_contiguous(wcodes) || !is_contiguous(wsf) || !is_contiguous(gs)) invalid("nvfp4 operand: not contiguous");
    if (numel_of(wcodes) >= INT32_MAX) invalid("nvfp4 operand: more elements than the kernels can index");
    const fl_tensor_view_impl_t &a = deref(a_h);
    check_activation(a, device, "the left operand");
    if (a.shape.back() != k) invalid("the two operands disagree about k");
    const fl_tensor_view_impl_t &out = deref(out_h);
    check_result(out, a, rows, device);
    if (act != FL_ACT_NONE && act != FL_ACT_GELU_TANH) invalid("unknown activation");
    const fl_tensor_view_impl_t *bias = bias_h ? &deref(bias_h) : nullptr;
    const fl_tensor_view_impl_t *residual = residual_h ? &deref(residual_h) : nullptr;
    if (bias) {
      if (device_of(*bias) != device || dtype_of(*bias) != dtype_of(out) || numel_of(*bias) != rows ||
          !is_contiguous(*bias)) {
        invalid("the bias is not a contiguous (rows) vector of out's type on the weight's device");
      }
    }
    if (residual) {
      if (device_of(*residual) != device || dtype_of(*residual) != dtype_of(out) || !is_contiguous(*residual)) {
        invalid("the residual is not contiguous, of out's type, on the weight's device");
      }
      check_shape(*residual, out.shape, "the residual");
    }
    if (device != FL_DEVICE_CUDA) invalid("the nvfp4 operand is on a device with no NVFP4 kernels");
    check_tiles(rows, k, 32);
    require_kernels();
    check_earlier_kernel_status();

    const int64_t m64 = leading_rows(a);
    if (m64 == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("the left operand has more rows than the kernels can index");
    const int m = static_cast<int>(m64);
    const int is_bf16 = dtype_of(a) == FL_DTYPE_BFLOAT16;

    Scratch scratch;
    const size_t xcodes_off = scratch.reserve(static_cast<size_t>(m) * k / 2);
    const size_t sfa_bytes = static_cast<size_t>(sf_tiled_bytes(m, k, 0));
    const size_t sfb_bytes = static_cast<size_t>(sf_tiled_bytes(rows, k, 1));  // one spare row group: a
    const size_t sfa_off = scratch.reserve(sfa_bytes);                          // tile may read past the last
    const size_t sfb_off = scratch.reserve(sfb_bytes);
    size_t w_off = 0;
    const bool w_misaligned = !aligned16(raw_ptr(wcodes));
    if (w_misaligned) w_off = scratch.reserve(static_cast<size_t>(rows) * k / 2);
    uint8_t *base = scratch.commit();

    // One launch: the activation's codes and scale factors, the weight's block scales re-tiled,
    // zeros in the padding of both (four launches with a gap each before: 1 805 -> 2 005 TFLOP/s on C3).
    cuda_check(nvfp4_prepare(raw_ptr(a), is_bf16, m, k, base + xcodes_off, base + sfa_off,
                             reinterpret_cast<const uint8_t *>(raw_ptr(wsf)), rows, 1, base + sfb_off, 0),
               "quantising the activation and re-tiling the block scales");
    const void *w_ptr = raw_ptr(wcodes);
    if (w_misaligned) {
      cuda_check(cudaMemcpyAsync(base + w_off, w_ptr, static_cast<size_t>(rows) * k / 2, cudaMemcpyDeviceToDevice, 0),
                 "staging the weight");
      w_ptr = base + w_off;
    }
    Epilogue ep;
    ep.global_scale = reinterpret_cast<const float *>(raw_ptr(gs));
    ep.bias = bias ? raw_ptr(*bias) : nullptr;
    if (residual) {
      ep.residual = raw_ptr(*residual);
      ep.residual_rows = m;
      ep.residual_ld = rows;
    }
    ep.act = act;
    run_gemm(kGemmNvf4, m, rows, k, base + xcodes_off, w_ptr, base + sfa_off, base + sfb_off, ep, is_bf16,
             raw_ptr(out));
    return clear_error();
  });
}

int32_t fl_quantize_fp8_rows(fl_tensor_view_t w_h, fl_tensor_view_t codes_h, fl_tensor_view_t scales_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &w = deref(w_h);
    const fl_tensor_view_impl_t &codes = deref(codes_h);
    const fl_tensor_view_impl_t &scales = deref(scales_h);
    if (dtype_of(w) != FL_DTYPE_FLOAT || w.shape.size() != 2 || !is_contiguous(w)) invalid("w is not a contiguous <float>(rows, k)");
    if (dtype_of(codes) != FL_DTYPE_FP8E4M3 || codes.shape != w.shape || !is_contiguous(codes)) invalid("codes is not a contiguous <fp8e4m3>(rows, k)");
    if (dtype_of(scales) != FL_DTYPE_FLOAT || numel_of(scales) != w.shape[0] || !is_contiguous(scales)) invalid("scales is not a contiguous <float>(rows)");
    if (device_of(w) != FL_DEVICE_CUDA || device_of(codes) != FL_DEVICE_CUDA || device_of(scales) != FL_DEVICE_CUDA) invalid("the operands are not all on cuda");
    require_kernels();
    if (numel_of(w) == 0) return clear_error();
    cuda_check(quantize_fp8_rows_f32(reinterpret_cast<const float *>(raw_ptr(w)), w.shape[0], w.shape[1], raw_ptr(codes),
                                     reinterpret_cast<float *>(raw_ptr(scales)), 0),
               "quantising");
    return clear_error();
  });
}

int32_t fl_quantize_fp8_activation(fl_tensor_view_t a_h, fl_tensor_view_t codes_h, fl_tensor_view_t scales_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &a = deref(a_h);
    const fl_tensor_view_impl_t &codes = deref(codes_h);
    const fl_tensor_view_impl_t &scales = deref(scales_h);
    if (!is_half_type(dtype_of(a)) || a.shape.size() != 2 || !is_contiguous(a)) invalid("a is not a contiguous 16-bit (m, k)");
    if (dtype_of(codes) != FL_DTYPE_FP8E4M3 || codes.shape != a.shape || !is_contiguous(codes)) invalid("codes is not a contiguous <fp8e4m3>(m, k)");
    if (dtype_of(scales) != FL_DTYPE_FLOAT || numel_of(scales) != a.shape[0] || !is_contiguous(scales)) invalid("scales is not a contiguous <float>(m)");
    if (device_of(a) != FL_DEVICE_CUDA || device_of(codes) != FL_DEVICE_CUDA || device_of(scales) != FL_DEVICE_CUDA) invalid("the operands are not all on cuda");
    require_kernels();
    if (numel_of(a) == 0) return clear_error();
    cuda_check(quantize_fp8_act(raw_ptr(a), dtype_of(a) == FL_DTYPE_BFLOAT16, a.shape[0], a.shape[1], raw_ptr(codes),
                                reinterpret_cast<float *>(raw_ptr(scales)), 0),
               "quantising");
    return clear_error();
  });
}

namespace {
// Elements between the rows of a (groups, k) modulation tensor (k for a plain vector).
int64_t group_pitch(const fl_tensor_view_impl_t *v, int k) {
  if (!v || v->shape.size() < 2 || v->shape[0] == 1) return k;
  return v->stride[0];
}
}  // namespace

int32_t fl_fp8_layernorm_quantize(fl_tensor_view_t x_h, fl_tensor_view_t scale_h, fl_tensor_view_t shift_h, float eps,
                                  fl_tensor_view_t codes_h, fl_tensor_view_t row_scales_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &x = deref(x_h);
    const fl_tensor_view_impl_t &codes = deref(codes_h);
    const fl_tensor_view_impl_t &row_scales = deref(row_scales_h);
    if (!is_half_type(dtype_of(x)) || x.shape.size() < 2 || !is_contiguous(x)) {
      invalid("x is not a contiguous <float16> or <bfloat16> tensor of at least two dimensions");
    }
    if (dtype_of(codes) != FL_DTYPE_FP8E4M3 || codes.shape != x.shape || !is_contiguous(codes)) {
      invalid("codes is not a contiguous <fp8e4m3> tensor of x's shape");
    }
    const int64_t m64 = leading_rows(x);
    const int k = x.shape.back();
    if (dtype_of(row_scales) != FL_DTYPE_FLOAT || numel_of(row_scales) != m64 || !is_contiguous(row_scales)) {
      invalid("row_scales is not a contiguous <float> tensor of one value per row of x");
    }
    if (!(eps >= 0.0f)) invalid("eps is negative or not a number");
    int64_t groups = 1;
    const fl_tensor_view_impl_t *mods[2] = {scale_h ? &deref(scale_h) : nullptr, shift_h ? &deref(shift_h) : nullptr};
    for (const fl_tensor_view_impl_t *v : mods) {
      if (!v) continue;
      // (k), or (groups, k) whose rows may be slices of a wider tensor (any row stride, unit
      // column stride): the modulation vectors are chunks of one projection's output.
      if (dtype_of(*v) != dtype_of(x) || v->shape.empty() || v->shape.size() > 2 || v->shape.back() != k ||
          (k > 1 && v->stride.back() != 1)) {
        invalid("scale/shift is not a (k) or (groups, k) tensor of x's type with contiguous rows");
      }
      const int64_t g = v->shape.size() == 2 ? v->shape[0] : 1;
      if (groups != 1 && g != 1 && g != groups) invalid("scale and shift disagree about the number of groups");
      if (g != 1) groups = g;
    }
    for (const fl_tensor_view_impl_t *v : mods) {
      if (v && groups != 1 && (v->shape.size() == 2 ? v->shape[0] : 1) != groups) {
        invalid("scale and shift disagree about the number of groups");
      }
    }
    if (m64 > 0 && m64 % groups != 0) invalid("the rows of x do not divide into the groups of scale/shift");
    for (const fl_tensor_view_impl_t *v : {&x, &codes, &row_scales}) {
      if (device_of(*v) != FL_DEVICE_CUDA) invalid("the operands are not all on cuda");
    }
    for (const fl_tensor_view_impl_t *v : mods) {
      if (v && device_of(*v) != FL_DEVICE_CUDA) invalid("the operands are not all on cuda");
    }
    require_kernels();
    if (m64 == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("x has more rows than the kernels can index");
    cuda_check(ln_modulate_quantize_fp8(raw_ptr(x), dtype_of(x) == FL_DTYPE_BFLOAT16, static_cast<int>(m64), k,
                                        mods[0] ? raw_ptr(*mods[0]) : nullptr, group_pitch(mods[0], k),
                                        mods[1] ? raw_ptr(*mods[1]) : nullptr, group_pitch(mods[1], k),
                                        static_cast<int>(m64 / groups), eps, raw_ptr(codes),
                                        reinterpret_cast<float *>(raw_ptr(row_scales)), 0),
               "layer norm and quantisation");
    return clear_error();
  });
}

namespace {

// fl_fp8_linear_quantized (out_h) and fl_fp8_linear_quantized_scatter (dests): one of the two is given.
int32_t fp8_linear_quantized_impl(fl_tensor_view_t codes_h, fl_tensor_view_t row_scales_h, fl_tensor_view_t data_h,
                                  fl_tensor_view_t scales_h, fl_tensor_view_t bias_h, fl_tensor_view_t residual_h,
                                  int32_t act, fl_tensor_view_t out_h, const fl_tensor_view_t *dests, int32_t n_dest,
                                  int32_t col0, int32_t rows_per_group = 0) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &weight = deref(data_h);
    const fl_tensor_view_impl_t &scales = deref(scales_h);
    if (rows_per_group == 0) {
      check_fp8_weight(weight, scales, /*per_channel_ok=*/true);
    } else {
      // Row groups: the scales (and the bias) are (groups, rows) matrices, row g for the rows of group g.
      if (dtype_of(weight) != FL_DTYPE_FP8E4M3 || weight.shape.size() != 2 || !is_contiguous(weight) ||
          numel_of(weight) >= INT32_MAX) {
        invalid("fp8 operand: data is not a contiguous <fp8e4m3>(rows, k)");
      }
      if (rows_per_group < 0 || rows_per_group % 256 != 0) invalid("rows_per_group is not a positive multiple of 256");
      if (!out_h) invalid("row groups and a scattered result do not combine");
    }
    const fl_device_type_t device = device_of(weight);
    const int rows = weight.shape[0];
    const int k = weight.shape[1];
    const fl_tensor_view_impl_t &a = deref(codes_h);
    const fl_tensor_view_impl_t &row_scales = deref(row_scales_h);
    if (dtype_of(a) != FL_DTYPE_FP8E4M3 || a.shape.size() < 2 || !is_contiguous(a) || device_of(a) != device) {
      invalid("the left operand is not a contiguous <fp8e4m3> tensor of at least two dimensions on the weight's device");
    }
    if (a.shape.back() != k) invalid("the two operands disagree about k");
    const int64_t m64 = leading_rows(a);
    if (dtype_of(row_scales) != FL_DTYPE_FLOAT || numel_of(row_scales) != m64 || !is_contiguous(row_scales) ||
        device_of(row_scales) != device) {
      invalid("row_scales is not a contiguous <float> tensor of one value per row on the weight's device");
    }
    std::vector<int32_t> out_shape(a.shape.begin(), a.shape.end());
    out_shape.back() = rows;
    ScatterDests sd;
    fl_dtype_t out_dtype;
    if (out_h) {
      const fl_tensor_view_impl_t &out = deref(out_h);
      if (!is_half_type(dtype_of(out)) || device_of(out) != device || !is_contiguous(out)) {
        invalid("out is not a contiguous <float16> or <bfloat16> tensor on the weight's device");
      }
      check_shape(out, out_shape, "out");
      out_dtype = dtype_of(out);
      sd.first = raw_ptr(out);
    } else {
      if (!dests || n_dest < 1) invalid("scatter: between 1 and " + std::to_string(kMaxGemmOutputs) + " destinations are needed");
      out_dtype = dtype_of(deref(dests[0]));
      if (!is_half_type(out_dtype)) invalid("scatter: the destinations are not <float16> or <bfloat16>");
      sd = check_scatter_dests(dests, n_dest, col0, rows, a.shape, out_dtype, device);
    }
    if (act != FL_ACT_NONE && act != FL_ACT_GELU_TANH) invalid("unknown activation");
    const fl_tensor_view_impl_t *bias = bias_h ? &deref(bias_h) : nullptr;
    const fl_tensor_view_impl_t *residual = residual_h ? &deref(residual_h) : nullptr;
    const int64_t groups = rows_per_group > 0 ? (m64 + rows_per_group - 1) / rows_per_group : 1;
    if (rows_per_group > 0 && (dtype_of(scales) != FL_DTYPE_FLOAT || numel_of(scales) != groups * rows || !is_contiguous(scales) ||
                               device_of(scales) != device)) {
      invalid("the scales are not a contiguous <float>(groups, rows) matrix on the weight's device");
    }
    if (bias) {
      if (device_of(*bias) != device || dtype_of(*bias) != out_dtype || numel_of(*bias) != groups * rows ||
          !is_contiguous(*bias)) {
        invalid(rows_per_group > 0 ? "the bias is not a contiguous (groups, rows) matrix of out's type on the weight's device"
                                   : "the bias is not a contiguous (rows) vector of out's type on the weight's device");
      }
    }
    if (residual) {
      if (device_of(*residual) != device || dtype_of(*residual) != out_dtype || !is_contiguous(*residual)) {
        invalid("the residual is not contiguous, of out's type, on the weight's device");
      }
      check_shape(*residual, out_shape, "the residual");
    }
    if (device != FL_DEVICE_CUDA) invalid("the fp8 operand is on a device with no FP8 kernels");
    check_tiles(rows, k, 16);
    require_kernels();
    check_earlier_kernel_status();
    if (m64 == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("the left operand has more rows than the kernels can index");
    const int m = static_cast<int>(m64);

    // TMA wants 16-byte aligned bases; a view that starts elsewhere is staged.
    Scratch scratch;
    size_t a_off = 0, w_off = 0;
    const bool a_misaligned = !aligned16(raw_ptr(a));
    const bool w_misaligned = !aligned16(raw_ptr(weight));
    if (a_misaligned) a_off = scratch.reserve(static_cast<size_t>(m) * k);
    if (w_misaligned) w_off = scratch.reserve(static_cast<size_t>(rows) * k);
    const void *a_ptr = raw_ptr(a);
    const void *w_ptr = raw_ptr(weight);
    if (a_misaligned || w_misaligned) {
      uint8_t *base = scratch.commit();
      if (a_misaligned) {
        cuda_check(cudaMemcpyAsync(base + a_off, a_ptr, static_cast<size_t>(m) * k, cudaMemcpyDeviceToDevice, 0),
                   "staging the left operand");
        a_ptr = base + a_off;
      }
      if (w_misaligned) {
        cuda_check(cudaMemcpyAsync(base + w_off, w_ptr, static_cast<size_t>(rows) * k, cudaMemcpyDeviceToDevice, 0),
                   "staging the weight");
        w_ptr = base + w_off;
      }
    }
    Epilogue ep;
    ep.row_scale = reinterpret_cast<const float *>(raw_ptr(row_scales));
    ep.col_scale = reinterpret_cast<const float *>(raw_ptr(scales));
    ep.col_scale_scalar = numel_of(scales) == 1 ? 1 : 0;
    ep.bias = bias ? raw_ptr(*bias) : nullptr;
    if (residual) {
      ep.residual = raw_ptr(*residual);
      ep.residual_rows = m;
      ep.residual_ld = rows;
    }
    ep.act = act;
    ep.rows_per_group = rows_per_group;
    if (!out_h) {
      ep.out_ld = sd.ld;
      ep.out_col0 = col0;
      for (int i = 0; i < sd.num_extra; ++i) ep.extra_out[ep.num_extra_out++] = sd.extra[i];
    }
    if (out_h && rows_per_group == 0 &&
        try_fewrow_q8(reinterpret_cast<const uint8_t *>(a_ptr), ep.row_scale, m, rows, k, w_ptr, ep,
                               out_dtype == FL_DTYPE_BFLOAT16, sd.first, status_word())) {
      return clear_error();
    }
    run_gemm(kGemmE4M3, m, rows, k, a_ptr, w_ptr, nullptr, nullptr, ep, out_dtype == FL_DTYPE_BFLOAT16, sd.first);
    return clear_error();
  });
}

}  // namespace

int32_t fl_fp8_linear_quantized(fl_tensor_view_t codes_h, fl_tensor_view_t row_scales_h, fl_tensor_view_t data_h,
                                fl_tensor_view_t scales_h, fl_tensor_view_t bias_h, fl_tensor_view_t residual_h,
                                int32_t act, fl_tensor_view_t out_h) {
  if (!out_h) return guard([&]() -> int32_t { invalid("out is null"); });
  return fp8_linear_quantized_impl(codes_h, row_scales_h, data_h, scales_h, bias_h, residual_h, act, out_h, nullptr, 0, 0);
}

int32_t fl_fp8_linear_quantized_grouped(fl_tensor_view_t codes_h, fl_tensor_view_t row_scales_h, fl_tensor_view_t data_h,
                                        fl_tensor_view_t scales_h, fl_tensor_view_t bias_h, fl_tensor_view_t residual_h,
                                        int32_t act, int32_t rows_per_group, fl_tensor_view_t out_h) {
  if (!out_h) return guard([&]() -> int32_t { invalid("out is null"); });
  if (rows_per_group <= 0) return guard([&]() -> int32_t { invalid("rows_per_group is not a positive multiple of 256"); });
  return fp8_linear_quantized_impl(codes_h, row_scales_h, data_h, scales_h, bias_h, residual_h, act, out_h, nullptr, 0, 0,
                                   rows_per_group);
}

int32_t fl_fp8_linear_quantized_scatter(fl_tensor_view_t codes_h, fl_tensor_view_t row_scales_h, fl_tensor_view_t data_h,
                                        fl_tensor_view_t scales_h, fl_tensor_view_t bias_h, fl_tensor_view_t residual_h,
                                        int32_t act, const fl_tensor_view_t *dests, int32_t n_dest, int32_t col0) {
  return fp8_linear_quantized_impl(codes_h, row_scales_h, data_h, scales_h, bias_h, residual_h, act, nullptr, dests, n_dest, col0);
}

int32_t fl_fp8_swiglu_quantize(fl_tensor_view_t x_h, fl_tensor_view_t codes_h, fl_tensor_view_t row_scales_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &x = deref(x_h);
    const fl_tensor_view_impl_t &codes = deref(codes_h);
    const fl_tensor_view_impl_t &row_scales = deref(row_scales_h);
    if (!is_half_type(dtype_of(x)) || x.shape.size() < 2 || !is_contiguous(x) || x.shape.back() % 2 != 0) {
      invalid("x is not a contiguous <float16> or <bfloat16> tensor of at least two dimensions with an even last one");
    }
    std::vector<int32_t> want(x.shape.begin(), x.shape.end());
    want.back() /= 2;
    if (dtype_of(codes) != FL_DTYPE_FP8E4M3 || codes.shape != want || !is_contiguous(codes)) {
      invalid("codes is not a contiguous <fp8e4m3> tensor of x's shape with half the last dimension");
    }
    const int64_t m64 = leading_rows(x);
    if (dtype_of(row_scales) != FL_DTYPE_FLOAT || numel_of(row_scales) != m64 || !is_contiguous(row_scales)) {
      invalid("row_scales is not a contiguous <float> tensor of one value per row of x");
    }
    for (const fl_tensor_view_impl_t *v : {&x, &codes, &row_scales}) {
      if (device_of(*v) != FL_DEVICE_CUDA) invalid("the operands are not all on cuda");
    }
    require_kernels();
    if (m64 == 0 || want.back() == 0) return clear_error();
    if (m64 > INT32_MAX) invalid("x has more rows than the kernels can index");
    cuda_check(swiglu_quantize_fp8(raw_ptr(x), dtype_of(x) == FL_DTYPE_BFLOAT16, static_cast<int>(m64), want.back(),
                                   raw_ptr(codes), reinterpret_cast<float *>(raw_ptr(row_scales)), 0),
               "swiglu and quantisation");
    return clear_error();
  });
}

int32_t fl_qk_norm_rope(fl_tensor_view_t qkv_h, fl_tensor_view_t q_weight_h, fl_tensor_view_t k_weight_h,
                        fl_tensor_view_t cos_h, fl_tensor_view_t sin_h, float eps, int32_t heads) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &qkv = deref(qkv_h);
    const fl_tensor_view_impl_t &cos = deref(cos_h);
    const fl_tensor_view_impl_t &sin = deref(sin_h);
    if (!is_half_type(dtype_of(qkv)) || qkv.shape.size() < 2 || !is_contiguous(qkv)) {
      invalid("qkv is not a contiguous <float16> or <bfloat16> tensor of at least two dimensions");
    }
    if (heads <= 0 || qkv.shape.back() % (3 * heads) != 0) invalid("qkv's last dimension is not 3 * heads * head_dim");
    const int head_dim = qkv.shape.back() / (3 * heads);
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) invalid("head_dim is not 64, 128 or 256");
    for (const fl_tensor_view_impl_t *v : {&cos, &sin}) {
      if (dtype_of(*v) != FL_DTYPE_FLOAT || v->shape.size() != 2 || v->shape[1] != head_dim / 2 || !is_contiguous(*v)) {
        invalid("cos/sin is not a contiguous <float>(tokens, head_dim / 2)");
      }
    }
    if (cos.shape != sin.shape) invalid("cos and sin differ in shape");
    const int tokens = cos.shape[0];
    const int64_t rows = leading_rows(qkv);
    if (tokens <= 0 || rows % tokens != 0) invalid("the rows of qkv are not whole sequences of cos/sin's tokens");
    const fl_tensor_view_impl_t *weights[2] = {q_weight_h ? &deref(q_weight_h) : nullptr,
                                               k_weight_h ? &deref(k_weight_h) : nullptr};
    for (const fl_tensor_view_impl_t *w : weights) {
      if (w && (dtype_of(*w) != dtype_of(qkv) || numel_of(*w) != head_dim || !is_contiguous(*w) ||
                device_of(*w) != FL_DEVICE_CUDA)) {
        invalid("a norm weight is not a contiguous (head_dim) vector of qkv's type on cuda");
      }
    }
    if (!(eps >= 0.0f)) invalid("eps is negative or not a number");
    for (const fl_tensor_view_impl_t *v : {&qkv, &cos, &sin}) {
      if (device_of(*v) != FL_DEVICE_CUDA) invalid("the operands are not all on cuda");
    }
    for (const fl_tensor_view_impl_t *v : {&qkv, &cos, &sin}) {
      if (!aligned16(raw_ptr(*v))) invalid("qkv, cos and sin have to start on 16-byte boundaries");
    }
    for (const fl_tensor_view_impl_t *w : weights) {
      if (w && !aligned16(raw_ptr(*w))) invalid("a norm weight does not start on a 16-byte boundary");
    }
    require_kernels();
    if (rows == 0) return clear_error();
    if (rows > INT32_MAX) invalid("qkv has more rows than the kernel can index");
    cuda_check(qk_norm_rope(raw_ptr(qkv), dtype_of(qkv) == FL_DTYPE_BFLOAT16, rows, heads, head_dim, tokens,
                            weights[0] ? raw_ptr(*weights[0]) : nullptr, weights[1] ? raw_ptr(*weights[1]) : nullptr,
                            reinterpret_cast<const float *>(raw_ptr(cos)), reinterpret_cast<const float *>(raw_ptr(sin)), eps, 0),
               "q/k norm and rotation");
    ++g_block_launches;
    return clear_error();
  });
}

// flint/capi.h:532-544, every mask of flint/capi.h:118-133; the checks are those of
// flint/operators.cc:108-146.
int32_t fl_attention(fl_operators_t operators, fl_tensor_view_t q_h, fl_tensor_view_t k_h, fl_tensor_view_t v_h,
                     fl_mask_type_t mask_type, int32_t block_size, fl_tensor_view_t out_h) {
  return guard([&]() -> int32_t {
    if (!operators) invalid("operators is null");
    const fl_tensor_view_impl_t &q = deref(q_h);
    const fl_tensor_view_impl_t &k = deref(k_h);
    const fl_tensor_view_impl_t &v = deref(v_h);
    const fl_tensor_view_impl_t &out = deref(out_h);
    if (mask_type < FL_MASK_NONE || mask_type > FL_MASK_BLOCK_DIAGONAL) invalid("attention: unknown mask type");
    const bool block_mask = mask_type == FL_MASK_BLOCK_CAUSAL || mask_type == FL_MASK_BLOCK_DIAGONAL;
    if (!block_mask && block_size != 0) {
      invalid("attention: a block size of " + std::to_string(block_size) + " without a block mask");
    }
    if (block_mask && block_size <= 0) {
      invalid("attention: a block mask of " + std::to_string(block_size) + " keys a block");
    }
    for (const fl_tensor_view_impl_t *t : {&q, &k, &v, &out}) {
      if (t->shape.size() != 4) invalid("attention: q, k, v and out are four-dimensional");
      if (device_of(*t) != FL_DEVICE_CUDA) invalid("an operand is not on the operators' device");
      if (!is_half_type(dtype_of(*t)) || dtype_of(*t) != dtype_of(q)) {
        invalid("attention: this library takes <float16> or <bfloat16> operands of one type");
      }
      if (t->shape[3] > 1 && t->stride[3] != 1) invalid("attention: the last dimension is not contiguous");
    }
    const int batch = q.shape[0], heads = q.shape[1], q_len = q.shape[2], d = q.shape[3];
    const int kv_heads = k.shape[1], kv_len = k.shape[2];
    if (k.shape[0] != batch || k.shape[3] != d || v.shape != k.shape) invalid("attention: k and v disagree with q or each other");
    if (out.shape != q.shape) invalid("attention: out is not of q's shape");
    if (kv_heads <= 0 || heads % kv_heads != 0) invalid("attention: the query heads are not a multiple of the key-value heads");
    if (kv_len <= 0) invalid("attention: no keys");
    if (mask_type == FL_MASK_CAUSAL && kv_len < q_len) invalid("attention: keys too few for the causal mask");
    if (mask_type == FL_MASK_BLOCK_CAUSAL && kv_len < q_len) {
      invalid("attention: a block causal mask over " + std::to_string(kv_len) + " keys and " + std::to_string(q_len) +
              " queries, which leaves the first queries before every key");
    }
    if (mask_type == FL_MASK_BLOCK_DIAGONAL && kv_len != q_len) {
      invalid("attention: a block diagonal mask is self-attention, and this is " + std::to_string(q_len) +
              " queries over " + std::to_string(kv_len) + " keys");
    }
    require_kernels();
    check_earlier_kernel_status();
    if (batch == 0 || q_len == 0) return clear_error();

    AttentionArgs a = {};
    a.q = raw_ptr(q);
    a.k = raw_ptr(k);
    a.v = raw_ptr(v);
    a.out = raw_ptr(out);
    a.is_bf16 = dtype_of(q) == FL_DTYPE_BFLOAT16;
    a.batch = batch;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.q_len = q_len;
    a.kv_len = kv_len;
    a.head_dim = d;
    for (int i = 0; i < 3; ++i) {
      a.q_stride[i] = q.stride[i];
      a.k_stride[i] = k.stride[i];
      a.v_stride[i] = v.stride[i];
      a.out_stride[i] = out.stride[i];
    }
    a.mask_type = static_cast<int>(mask_type);
    a.block_size = block_size;
    a.status = status_word();
    a.stream = 0;
    const char *why = "";
    if (!attention_supported(a, &why)) invalid(std::string("attention: ") + why + " (not implemented in this library)");
    const AttentionPlan plan = attention_plan(a);
    Scratch scratch;
    if (!plan.v_direct) {  // v goes through its transposition
      const size_t vt_off = scratch.reserve(attention_scratch_bytes(batch, kv_heads, kv_len, d));
      a.v_transposed = scratch.commit() + vt_off;
    }
    cudaError_t e = attention(a, &why);
    if (e != cudaSuccess) cuda_check(e, (std::string("attention: ") + why).c_str());
    g_block_launches += plan.launches;
    return clear_error();
  });
}

int32_t fl_quantize_nvfp4(fl_tensor_view_t w_h, fl_tensor_view_t codes_h, fl_tensor_view_t block_scales_h,
                          fl_tensor_view_t global_scale_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &w = deref(w_h);
    const fl_tensor_view_impl_t &codes = deref(codes_h);
    const fl_tensor_view_impl_t &sf = deref(block_scales_h);
    const fl_tensor_view_impl_t &gs = deref(global_scale_h);
    if (dtype_of(w) != FL_DTYPE_FLOAT || w.shape.size() != 2 || !is_contiguous(w)) invalid("w is not a contiguous <float>(rows, k)");
    const int rows = w.shape[0], k = w.shape[1];
    if (k % 16 != 0) invalid("k is not a multiple of 16");
    if (dtype_of(codes) != FL_DTYPE_FP4E2M1X2 || codes.shape != std::vector<int32_t>{rows, k / 2} || !is_contiguous(codes)) invalid("codes is not a contiguous <fp4e2m1x2>(rows, k/2)");
    if (dtype_of(sf) != FL_DTYPE_FP8E4M3 || sf.shape != std::vector<int32_t>{rows, k / 16} || !is_contiguous(sf)) invalid("block_scales is not a contiguous <fp8e4m3>(rows, k/16)");
    if (dtype_of(gs) != FL_DTYPE_FLOAT || numel_of(gs) != 1) invalid("global_scale is not a single <float>");
    if (device_of(w) != FL_DEVICE_CUDA || device_of(codes) != FL_DEVICE_CUDA || device_of(sf) != FL_DEVICE_CUDA || device_of(gs) != FL_DEVICE_CUDA) invalid("the operands are not all on cuda");
    require_kernels();
    if (numel_of(w) == 0) return clear_error();
    Scratch scratch;
    const size_t word_off = scratch.reserve(256);
    uint8_t *base = scratch.commit();
    cuda_check(quantize_nvfp4_weight_f32(reinterpret_cast<const float *>(raw_ptr(w)), rows, k, raw_ptr(codes), raw_ptr(sf),
                                         reinterpret_cast<float *>(raw_ptr(gs)),
                                         reinterpret_cast<uint32_t *>(base + word_off), 0),
               "quantising");
    return clear_error();
  });
}

int32_t fl_tensor_data_borrow_device(void *device_ptr, fl_dtype_t dtype, int64_t numel, fl_tensor_data_t *out) {
  return guard([&]() {
    if (!out) invalid("out is null");
    if (!device_ptr) invalid("device_ptr is null");
    if (numel < 1) invalid("storage holds at least one element");
    const int64_t alignment = dtype_size(dtype);
    if (reinterpret_cast<uintptr_t>(device_ptr) % alignment != 0) {
      invalid("device_ptr is not aligned to its " + std::to_string(alignment) + "-byte elements");
    }
    auto *d = new fl_tensor_data_impl_t();
    d->ptr = device_ptr;
    d->numel = numel;
    d->dtype = dtype;
    d->device = FL_DEVICE_CUDA;
    d->owned = false;
    *out = d;
    return clear_error();
  });
}

int32_t fl_sm100_set_device(int32_t ordinal) {
  return guard([&]() {
    {
      // One process drives one GPU: the kernel modules cache per-process facts about the device
      // (its SM count, which kernels had their shared-memory limit raised), so a second device
      // is refused here instead of failing at some later launch.
      std::lock_guard<std::mutex> lock(g_mutex);
      if (g_dev.device_in_use >= 0 && g_dev.device_in_use != ordinal) {
        invalid("this process already runs on cuda device " + std::to_string(g_dev.device_in_use) +
                "; the library drives one device per process and the device has to be chosen before the first operation");
      }
    }
    cuda_check(cudaSetDevice(ordinal), "cudaSetDevice");
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      g_dev.probed = false;
      probe_locked();
    }
    return clear_error();
  });
}

int32_t fl_sm100_synchronize(int32_t *kernel_status) {
  return guard([&]() -> int32_t {
    cuda_check(cudaStreamSynchronize(0), "cudaStreamSynchronize");
    uint32_t code = 0;
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      sweep_returning_locked(true);
      if (g_dev.status_host) {
        code = *reinterpret_cast<volatile uint32_t *>(g_dev.status_host);
        *reinterpret_cast<volatile uint32_t *>(g_dev.status_host) = 0;
      }
    }
    // fl_fp8_linear_static()'s kernels report through a word of their own, in the static array.
    if (code == 0) code = take_static_status();
    if (kernel_status) *kernel_status = static_cast<int32_t>(code);
    if (code != 0) rezero_stream_k_counters();
    if (code != 0) aborted("a kernel gave up on a bounded wait (status " + std::to_string(code) + ")");
    return clear_error();
  });
}

int32_t fl_sm100_gemm_timing(int32_t enable) {
  return guard([&]() {
    g_timing.enabled = enable != 0;
    return clear_error();
  });
}

int32_t fl_sm100_gemm_timing_read(double *total_ms, int64_t *launches) {
  return guard([&]() {
    if (!total_ms || !launches) invalid("out is null");
    cuda_check(cudaStreamSynchronize(0), "cudaStreamSynchronize");
    double sum = 0.0;
    for (auto &ev : g_timing.used) {
      float ms = 0.0f;
      cuda_check(cudaEventElapsedTime(&ms, ev.first, ev.second), "cudaEventElapsedTime");
      sum += ms;
      g_timing.spare.push_back(ev);
    }
    *launches = static_cast<int64_t>(g_timing.used.size());
    *total_ms = sum;
    g_timing.used.clear();
    return clear_error();
  });
}

int32_t fl_sm100_few_rows_plan(int32_t m, int32_t n, int32_t k, int32_t weight_bytes, int32_t activation_bytes,
                               int32_t has_residual, int32_t *plan) {
  return guard([&]() -> int32_t {
    if (!plan) invalid("plan is null");
    if ((weight_bytes != 1 && weight_bytes != 2) || (activation_bytes != 1 && activation_bytes != 2)) {
      invalid("weight_bytes and activation_bytes are 1 or 2");
    }
    for (int i = 0; i < 16; ++i) plan[i] = 0;
    skinny_plan(m, n, k, weight_bytes, activation_bytes, has_residual, plan);
    return clear_error();
  });
}

int32_t fl_sm100_few_rows_route(int32_t entry, int32_t m, int32_t n, int32_t k) {
  if (m < 1 || n < 1 || k < 1) return -1;
  switch (entry) {
    case 0: return fewrow_tc_route(m, n, k) ? 2 : m <= 16 ? 1 : 0;
    case 1: return fewrow_q8_route(m, n, k) ? 2 : m <= 4 ? 1 : 0;
    case 2: return fewrow_w16_route(m, n, k) ? 2 : m <= 16 ? 1 : 0;
    default: return -1;
  }
}

int32_t fl_sm100_gemm_plan(int32_t kind, int32_t m, int32_t n, int32_t k, int32_t sms, int32_t allow_stream_k, int32_t *plan) {
  return guard([&]() -> int32_t {
    if (!plan) invalid("plan is null");
    if (kind < kGemmF16 || kind > kGemmNvf4) invalid("kind is 0 (half), 1 (bfloat16), 2 (e4m3) or 3 (nvfp4)");
    if (m < 1 || n < 1 || k < 1 || sms < 2) invalid("m, n, k are positive and the device has at least two SMs");
    int out[8];
    gemm_plan(static_cast<GemmKind>(kind), m, n, k, sms, allow_stream_k, out);
    for (int i = 0; i < 8; ++i) plan[i] = out[i];
    return clear_error();
  });
}

int64_t fl_sm100_launch_count(void) {
  return g_gemm_launches.load() + g_block_launches.load() + helper_launch_count() + elementwise_launch_count() +
         general_matmul_launch_count();
}


}  // extern "C"

// ============================ fl_fp8_linear_static ============================================
//
// fl_fp8_linear for callers that must not allocate. Its activation scratch (the e4m3 codes, the
// per-row scales and the kernels' status word) is the file-scope device array below instead of the
// library's growable arena, so the call makes no cudaMalloc / cudaFree / cudaHostAlloc and none of
// the device-wide synchronisation those imply. Every GPU whose context loads this library holds
// the array (about 16.3 MiB) until the process exits.

namespace {

constexpr size_t kStaticStatusBytes = 256;                 // status word, padded
constexpr size_t kStaticMaxRows = 65536;                   // rows of the activation (m)
constexpr size_t kStaticMaxCodes = size_t(16) << 20;       // m * k, one byte per element
constexpr size_t kStaticScalesOffset = kStaticStatusBytes;
constexpr size_t kStaticCodesOffset = kStaticScalesOffset + kStaticMaxRows * sizeof(float);
constexpr size_t kStaticBytes = kStaticCodesOffset + kStaticMaxCodes;

// In host code this name is only a handle for cudaGetSymbolAddress(); it is not a device address
// and must never be handed to a kernel as one.
static __device__ __align__(256) uint8_t g_static_scratch[kStaticBytes];

constexpr int kStaticMaxDevices = 64;
uint8_t *g_static_base[kStaticMaxDevices] = {};
std::mutex g_static_mutex;

// The array's device address on the current device, looked up once per device with that device
// current. No allocation: the array was placed when the module was loaded.
uint8_t *static_scratch_base() {
  int dev = 0;
  cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= kStaticMaxDevices) aborted("device ordinal beyond the static scratch table");
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_base[dev]) {
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) {
      aborted(std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
    }
    g_static_base[dev] = static_cast<uint8_t *>(ptr);
  }
  return g_static_base[dev];
}

uint32_t take_static_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return 0;
  uint8_t *base;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    base = g_static_base[dev];
  }
  if (!base) return 0;  // no static call has run on this device
  uint32_t code = 0;
  cuda_check(cudaMemcpy(&code, base, sizeof(code), cudaMemcpyDeviceToHost), "reading the static status word");
  if (code != 0) cuda_check(cudaMemsetAsync(base, 0, sizeof(uint32_t), 0), "clearing the static status word");
  return code;
}

}  // namespace

extern "C" {

// Test hooks (declared in the header's last section). The first writes `code` into the static
// array's status word as a kernel that gave up would; the second runs a one-warp kernel that waits,
// with a limit of `polls` polls, on a barrier nothing ever arrives on and reports through the
// library's ordinary status word. Neither faults nor hangs anything.
int32_t fl_sm100_selftest_set_static_status(uint32_t code) {
  return guard([&]() -> int32_t {
    require_kernels();
    uint8_t *base = static_scratch_base();
    cuda_check(cudaMemcpy(base, &code, sizeof(code), cudaMemcpyHostToDevice), "writing the static status word");
    return clear_error();
  });
}

int32_t fl_sm100_selftest_wait_timeout(int32_t polls) {
  return guard([&]() -> int32_t {
    if (polls < 1 || polls > 4096) invalid("polls is between 1 and 4096");
    require_kernels();
    check_earlier_kernel_status();
    cuda_check(selftest_wait_timeout(static_cast<uint32_t>(polls), status_word(), 0), "launching the wait self-test");
    ++g_block_launches;
    return clear_error();
  });
}

int32_t fl_fp8_linear_static(fl_tensor_view_t a_h, fl_tensor_view_t data_h, fl_tensor_view_t scales_h,
                             fl_tensor_view_t bias_h, fl_tensor_view_t residual_h, int32_t act,
                             fl_tensor_view_t out_h) {
  return guard([&]() -> int32_t {
    const fl_tensor_view_impl_t &weight = deref(data_h);
    const fl_tensor_view_impl_t &scales = deref(scales_h);
    check_fp8_weight(weight, scales, /*per_channel_ok=*/true);
    const fl_device_type_t device = device_of(weight);
    const int rows = weight.shape[0];
    const int k = weight.shape[1];
    const fl_tensor_view_impl_t &a = deref(a_h);
    check_activation(a, device, "the left operand");
    if (a.shape.back() != k) invalid("the two operands disagree about k");
    const fl_tensor_view_impl_t &out = deref(out_h);
    check_result(out, a, rows, device);
    if (act != FL_ACT_NONE && act != FL_ACT_GELU_TANH) invalid("unknown activation");
    const fl_tensor_view_impl_t *bias = bias_h ? &deref(bias_h) : nullptr;
    const fl_tensor_view_impl_t *residual = residual_h ? &deref(residual_h) : nullptr;
    if (bias) {
      if (device_of(*bias) != device || dtype_of(*bias) != dtype_of(out) || numel_of(*bias) != rows ||
          !is_contiguous(*bias)) {
        invalid("the bias is not a contiguous (rows) vector of out's type on the weight's device");
      }
    }
    if (residual) {
      if (device_of(*residual) != device || dtype_of(*residual) != dtype_of(out) || !is_contiguous(*residual)) {
        invalid("the residual is not contiguous, of out's type, on the weight's device");
      }
      check_shape(*residual, out.shape, "the residual");
    }
    if (device != FL_DEVICE_CUDA) invalid("the fp8 operand is on a device with no FP8 kernels");
    check_tiles(rows, k, 16);
    require_kernels();

    const int64_t m64 = leading_rows(a);
    if (m64 == 0) return clear_error();
    // The limits of the fixed scratch, refused before anything is launched.
    if (m64 > static_cast<int64_t>(kStaticMaxRows)) {
      invalid("fl_fp8_linear_static: " + std::to_string(m64) + " activation rows exceed the static scratch's " +
              std::to_string(kStaticMaxRows) + "; use fl_fp8_linear");
    }
    if (m64 * k > static_cast<int64_t>(kStaticMaxCodes)) {
      invalid("fl_fp8_linear_static: m * k = " + std::to_string(m64 * k) + " exceeds the static scratch's " +
              std::to_string(kStaticMaxCodes) + " elements; use fl_fp8_linear");
    }
    // The ordinary entry point stages a misaligned weight through its arena; there is no room
    // set aside for that here.
    if (!aligned16(raw_ptr(weight))) {
      invalid("fl_fp8_linear_static: the weight's first element is not 16-byte aligned; use fl_fp8_linear");
    }
    const int m = static_cast<int>(m64);
    const int is_bf16 = dtype_of(a) == FL_DTYPE_BFLOAT16;

    uint8_t *base = static_scratch_base();
    uint32_t *status = reinterpret_cast<uint32_t *>(base);
    float *row_scales = reinterpret_cast<float *>(base + kStaticScalesOffset);
    uint8_t *codes = base + kStaticCodesOffset;

    // The array keeps whatever the last call left in it. The previous call's status word is read
    // back first (a 4-byte copy that waits for the stream), then cleared for this call; codes and
    // scales are fully overwritten by the quantiser for the m x k in use, so need no clearing.
    uint32_t previous = 0;
    cuda_check(cudaMemcpy(&previous, status, sizeof(previous), cudaMemcpyDeviceToHost), "reading the static status word");
    cuda_check(cudaMemsetAsync(status, 0, sizeof(uint32_t), 0), "clearing the static status word");
    if (previous != 0) {
      aborted("the previous fl_fp8_linear_static call's kernel gave up on a bounded wait (status " +
              std::to_string(previous) + ")");
    }

    cuda_check(quantize_fp8_act(raw_ptr(a), is_bf16, m, k, codes, row_scales, 0), "quantising the activation");

    {
      Epilogue ep;
      ep.col_scale = reinterpret_cast<const float *>(raw_ptr(scales));
      ep.col_scale_scalar = numel_of(scales) == 1 ? 1 : 0;
      ep.bias = bias ? raw_ptr(*bias) : nullptr;
      if (residual) {
        ep.residual = raw_ptr(*residual);
        ep.residual_rows = m;
        ep.residual_ld = rows;
      }
      ep.act = act;
      if (try_fewrow_q8(codes, row_scales, m, rows, k, raw_ptr(weight), ep, is_bf16, raw_ptr(out), status)) return clear_error();
    }

    GemmArgs g{};
    g.kind = kGemmE4M3;
    g.m = m;
    g.n = rows;
    g.k = k;
    g.a = codes;
    g.b = raw_ptr(weight);
    g.row_scale = row_scales;
    g.col_scale = reinterpret_cast<const float *>(raw_ptr(scales));
    g.col_scale_scalar = numel_of(scales) == 1 ? 1 : 0;
    g.bias = bias ? raw_ptr(*bias) : nullptr;
    if (residual) {
      g.residual = raw_ptr(*residual);
      g.residual_rows = m;
      g.residual_ld = rows;
    }
    g.act = act;
    g.out_bf16 = is_bf16;
    g.out = raw_ptr(out);
    g.status = status;
    g.stream = 0;
    const char *why = "";
    cudaError_t e = launch_gemm(g, &why);
    if (e != cudaSuccess) aborted(std::string("GEMM launch: ") + why + " (" + cudaGetErrorString(e) + ")");
    ++g_gemm_launches;
    return clear_error();
  });
}

}  // extern "C"
