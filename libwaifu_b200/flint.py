"""Host-side mirror of the reference's safe wrapper over the flint C ABI, for the quantized-linear
path only: ``Tensor`` (waifu/src/flint/tensor.rs), ``fp8_available`` (waifu/src/flint/fp8.rs:41-49)
and ``functional.fp8_matmul`` / ``fp8_matmul_add`` (waifu/src/flint/functional.rs:653-703), plus the
additive ``fp8_linear`` / ``nvfp4_linear``. Everything goes through ``libflint_sm100.so`` by ctypes,
exactly the calls a cgo/Rust/ctypes binding of the reference would make.

There is no fallback: if the CUDA library is missing, importing this module's ``lib()`` raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_int32, c_int64, c_void_p
from typing import Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libflint_sm100.so")

# flint/capi.h:48-54
FL_OK = 0
FL_ERROR_INVALID_ARG = 0x0100
FL_ERROR_ABORTED = 0x0102
FL_ERROR_OUT_OF_MEMORY = 0x0103


class DType:
    """flint/capi.h:84-94, plus the two appended values."""
    FLOAT = 1
    LONG = 2
    UINT8 = 3
    FLOAT16 = 4
    INT8 = 6
    BOOL = 8
    INT32 = 9
    FP8E4M3 = 10
    BFLOAT16 = 11
    FP4E2M1X2 = 12


DTYPE_SIZE = {DType.FLOAT: 4, DType.LONG: 8, DType.UINT8: 1, DType.FLOAT16: 2, DType.INT8: 1, DType.BOOL: 1,
              DType.INT32: 4, DType.FP8E4M3: 1, DType.BFLOAT16: 2, DType.FP4E2M1X2: 1}


class Device:
    """flint/capi.h:96-106"""
    CPU = 0
    CUDA = 1
    CUDA_HOST = 2
    METAL = 3
    VULKAN = 4
    UNKNOWN = 5


ACT_NONE = 0
ACT_GELU_TANH = 1


class FlintError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"flint error 0x{code:04x}: {message}")
        self.code = code
        self.message = message


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """The loaded C-ABI library. Raises if it has not been built -- there is no other path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m libwaifu_b200.build` (needs nvcc). "
            "The quantized-linear path has no CPU or library fallback.")
    L = ctypes.CDLL(LIB_PATH)
    V = c_void_p
    L.fl_init.restype = None
    L.fl_get_last_error_code.restype = c_int32
    L.fl_get_last_error_message.restype = c_char_p
    L.fl_is_device_available.argtypes = [c_int32, POINTER(c_int32)]
    L.fl_operators_create.argtypes = [c_int32, POINTER(V)]
    L.fl_operators_destroy.argtypes = [V]; L.fl_operators_destroy.restype = None
    L.fl_operators_get_device.argtypes = [V, POINTER(c_int32)]
    L.fl_tensor_data_create.argtypes = [c_int32, c_int32, c_int64, c_int32, POINTER(V)]
    L.fl_tensor_data_borrow.argtypes = [V, c_int32, c_int64, POINTER(V)]
    L.fl_tensor_data_borrow_device.argtypes = [V, c_int32, c_int64, POINTER(V)]
    L.fl_tensor_data_destroy.argtypes = [V]; L.fl_tensor_data_destroy.restype = None
    L.fl_tensor_data_get_host_ptr.argtypes = [V, POINTER(V)]
    L.fl_tensor_view_create.argtypes = [V, POINTER(c_int32), POINTER(c_int32), c_int32, c_int64, POINTER(V)]
    L.fl_tensor_view_destroy.argtypes = [V]; L.fl_tensor_view_destroy.restype = None
    L.fl_transfer.argtypes = [V, V, V]
    L.fl_transfer_async.argtypes = [V, c_int32, POINTER(V), POINTER(V)]; L.fl_transfer_async.restype = c_int32
    L.fl_transfer_wait.argtypes = [V]; L.fl_transfer_wait.restype = c_int32
    L.fl_transfer_wait_sync.argtypes = [V]; L.fl_transfer_wait_sync.restype = c_int32
    L.fl_transfer_destroy.argtypes = [V]; L.fl_transfer_destroy.restype = None
    L.fl_sm100_transfer_to_host_async.argtypes = [V, V, POINTER(V)]; L.fl_sm100_transfer_to_host_async.restype = c_int32
    for name in ("fl_copy", "fl_cast"):
        getattr(L, name).argtypes = [V, V, V]; getattr(L, name).restype = c_int32
    L.fl_fill.argtypes = [V, V, ctypes.c_float]; L.fl_fill.restype = c_int32
    L.fl_add.argtypes = [V, V, V, V]; L.fl_add.restype = c_int32
    L.fl_sm100_gemm_plan.argtypes = [c_int32] * 6 + [POINTER(c_int32)]; L.fl_sm100_gemm_plan.restype = c_int32
    L.fl_sm100_selftest_wait_timeout.argtypes = [c_int32]; L.fl_sm100_selftest_wait_timeout.restype = c_int32
    L.fl_sm100_selftest_set_static_status.argtypes = [ctypes.c_uint32]; L.fl_sm100_selftest_set_static_status.restype = c_int32
    L.fl_fp8_available.argtypes = [c_int32, POINTER(c_int32)]
    L.fl_nvfp4_available.argtypes = [c_int32, POINTER(c_int32)]
    L.fl_fp8_matmul.argtypes = [V, V, V, V]
    L.fl_matmul.argtypes = [V, V, V, V]; L.fl_matmul.restype = c_int32
    L.fl_matmul_add.argtypes = [V, V, V, V, V]; L.fl_matmul_add.restype = c_int32
    L.fl_fp8_matmul_add.argtypes = [V, V, V, V, V]
    L.fl_fp8_linear.argtypes = [V, V, V, V, V, c_int32, V]
    L.fl_nvfp4_linear.argtypes = [V, V, V, V, V, V, c_int32, V]
    L.fl_fp8_linear_static.argtypes = [V, V, V, V, V, c_int32, V]
    L.fl_fp8_linear_static.restype = c_int32
    L.fl_fp8_linear_scatter.argtypes = [V, V, V, V, V, c_int32, POINTER(V), c_int32, c_int32]
    L.fl_fp8_linear_scatter.restype = c_int32
    L.fl_fp8_linear_amax.argtypes = [V, V, V, V, V, c_int32, V, V]; L.fl_fp8_linear_amax.restype = c_int32
    L.fl_fp8_quantize_scatter.argtypes = [V, V, POINTER(V), c_int32, c_int32, V]; L.fl_fp8_quantize_scatter.restype = c_int32
    L.fl_fp8_linear_quantized_scatter.argtypes = [V, V, V, V, V, V, c_int32, POINTER(V), c_int32, c_int32]
    L.fl_fp8_linear_quantized_scatter.restype = c_int32
    L.fl_fp8_row_amax.argtypes = [V, V]; L.fl_fp8_row_amax.restype = c_int32
    L.fl_sm100_peer_exchange.argtypes = [POINTER(V), c_int32, c_int32, c_int32, V, c_int32]; L.fl_sm100_peer_exchange.restype = c_int32
    L.fl_sm100_ipc_export.argtypes = [V, V]; L.fl_sm100_ipc_export.restype = c_int32
    L.fl_sm100_ipc_import.argtypes = [V, c_int32, c_int64, POINTER(V)]; L.fl_sm100_ipc_import.restype = c_int32
    L.fl_quantize_fp8_rows.argtypes = [V, V, V]
    L.fl_quantize_fp8_activation.argtypes = [V, V, V]
    L.fl_quantize_nvfp4.argtypes = [V, V, V, V]
    L.fl_fp8_layernorm_quantize.argtypes = [V, V, V, ctypes.c_float, V, V]
    L.fl_fp8_layernorm_quantize.restype = c_int32
    L.fl_fp8_linear_quantized.argtypes = [V, V, V, V, V, V, c_int32, V]
    L.fl_fp8_linear_quantized.restype = c_int32
    L.fl_fp8_linear_quantized_grouped.argtypes = [V, V, V, V, V, V, c_int32, c_int32, V]
    L.fl_fp8_linear_quantized_grouped.restype = c_int32
    L.fl_fp8_swiglu_quantize.argtypes = [V, V, V]
    L.fl_fp8_swiglu_quantize.restype = c_int32
    L.fl_qk_norm_rope.argtypes = [V, V, V, V, V, ctypes.c_float, c_int32]
    L.fl_qk_norm_rope.restype = c_int32
    L.fl_attention.argtypes = [V, V, V, V, c_int32, c_int32, V]
    L.fl_attention.restype = c_int32
    L.fl_sm100_set_device.argtypes = [c_int32]
    L.fl_sm100_synchronize.argtypes = [POINTER(c_int32)]
    L.fl_sm100_launch_count.restype = c_int64
    L.fl_sm100_gemm_timing.argtypes = [c_int32]; L.fl_sm100_gemm_timing.restype = c_int32
    L.fl_sm100_gemm_timing_read.argtypes = [POINTER(ctypes.c_double), POINTER(c_int64)]
    L.fl_sm100_gemm_timing_read.restype = c_int32
    for name in ("fl_is_device_available", "fl_operators_create", "fl_operators_get_device", "fl_tensor_data_create",
                 "fl_tensor_data_borrow", "fl_tensor_data_borrow_device", "fl_tensor_data_get_host_ptr",
                 "fl_tensor_view_create", "fl_transfer", "fl_fp8_available", "fl_nvfp4_available", "fl_fp8_matmul",
                 "fl_fp8_matmul_add", "fl_fp8_linear", "fl_nvfp4_linear", "fl_quantize_fp8_rows",
                 "fl_quantize_fp8_activation", "fl_quantize_nvfp4", "fl_sm100_set_device", "fl_sm100_synchronize"):
        getattr(L, name).restype = c_int32
    L.fl_init()
    _lib = L
    return L


def check(code: int) -> None:
    """waifu/src/flint/mod.rs `check`: a non-zero code becomes an error carrying the message."""
    if code != FL_OK:
        raise FlintError(code, lib().fl_get_last_error_message().decode("utf-8", "replace"))


def init() -> None:
    lib()


def set_device(ordinal: int) -> None:
    check(lib().fl_sm100_set_device(int(ordinal)))


def synchronize() -> None:
    status = c_int32(0)
    check(lib().fl_sm100_synchronize(byref(status)))


class AllocHint:
    """fl_alloc_hint_t (flint/capi.h:137-147)."""
    ACTIVATION = 0
    WEIGHT = 1
    OTHER = 2
    TEMPORARY_WEIGHT = 3


def gemm_timing(enable: bool) -> None:
    check(lib().fl_sm100_gemm_timing(1 if enable else 0))


def gemm_timing_read():
    """(summed GEMM-kernel milliseconds, launches) since the last read; waits for the stream."""
    ms = ctypes.c_double(0.0)
    n = c_int64(0)
    check(lib().fl_sm100_gemm_timing_read(byref(ms), byref(n)))
    return ms.value, n.value


def launch_count() -> int:
    return int(lib().fl_sm100_launch_count())


def fp8_available(device: int = Device.CUDA) -> bool:
    """waifu/src/flint/fp8.rs:41-49: a device without the kernels answers no, never an error."""
    out = c_int32(0)
    try:
        check(lib().fl_fp8_available(int(device), byref(out)))
    except FlintError:
        return False
    return out.value != 0


def nvfp4_available(device: int = Device.CUDA) -> bool:
    out = c_int32(0)
    try:
        check(lib().fl_nvfp4_available(int(device), byref(out)))
    except FlintError:
        return False
    return out.value != 0


_operators = None


def operators():
    """The CUDA operators handle (process-wide, as flint's are: flint/operators.cc:696-793)."""
    global _operators
    if _operators is None:
        h = c_void_p()
        check(lib().fl_operators_create(Device.CUDA, byref(h)))
        _operators = h
    return _operators


def _contiguous_strides(shape: Sequence[int]):
    strides = []
    acc = 1
    for s in reversed(shape):
        strides.append(acc)
        acc *= max(int(s), 1)
    return list(reversed(strides))


class Tensor:
    """Storage plus one view of it (waifu/src/flint/tensor.rs). Owns its storage unless borrowed."""

    def __init__(self, data: c_void_p, view: c_void_p, shape, dtype: int, device: int, owns_data: bool = True,
                 keepalive=None):
        self._data = data
        self._view = view
        self._shape = tuple(int(s) for s in shape)
        self._dtype = dtype
        self._device = device
        self._owns = owns_data
        self._keepalive = keepalive

    # -- construction ---------------------------------------------------------------------
    @staticmethod
    def empty(shape: Sequence[int], dtype: int, device: int = Device.CUDA, hint: int = 0) -> "Tensor":
        """Uninitialised storage and a contiguous view of it. On the device it comes from the
        stream-ordered pool, except that `hint=AllocHint.WEIGHT` gives 2 MiB or more memory of its
        own (the kind fl_sm100_ipc_export can share)."""
        numel = int(np.prod(shape)) if len(shape) else 1
        data = c_void_p()
        check(lib().fl_tensor_data_create(device, dtype, max(numel, 1), int(hint), byref(data)))
        return Tensor._over(data, shape, _contiguous_strides(shape), 0, dtype, device, True)

    @staticmethod
    def _over(data, shape, stride, offset, dtype, device, owns, keepalive=None) -> "Tensor":
        nd = len(shape)
        sh = (c_int32 * max(nd, 1))(*[int(s) for s in shape])
        st = (c_int32 * max(nd, 1))(*[int(s) for s in stride])
        view = c_void_p()
        code = lib().fl_tensor_view_create(data, sh, st, nd, int(offset), byref(view))
        if code != FL_OK:
            if owns:
                lib().fl_tensor_data_destroy(data)
            check(code)
        return Tensor(data, view, shape, dtype, device, owns, keepalive)

    @staticmethod
    def from_numpy(arr: np.ndarray, dtype: int, device: int = Device.CUDA) -> "Tensor":
        """Copies a host array (whose bytes already are `dtype`'s encoding) to `device`."""
        arr = np.ascontiguousarray(arr)
        assert arr.dtype.itemsize == DTYPE_SIZE[dtype], (arr.dtype, dtype)
        host_data = c_void_p()
        check(lib().fl_tensor_data_borrow(arr.ctypes.data_as(c_void_p), dtype, max(arr.size, 1), byref(host_data)))
        host = Tensor._over(host_data, arr.shape, _contiguous_strides(arr.shape), 0, dtype, Device.CPU, True, arr)
        if device == Device.CPU:
            return host
        out = Tensor.empty(arr.shape, dtype, device)
        if arr.size:
            check(lib().fl_transfer(operators(), host.raw(), out.raw()))
        return out

    @staticmethod
    def from_device_ptr(ptr: int, shape: Sequence[int], dtype: int, keepalive=None, stride=None,
                        numel: Optional[int] = None) -> "Tensor":
        """A view over device memory someone else owns (a torch tensor's data_ptr())."""
        n = int(np.prod(shape)) if numel is None else int(numel)
        data = c_void_p()
        check(lib().fl_tensor_data_borrow_device(c_void_p(ptr), dtype, max(n, 1), byref(data)))
        st = _contiguous_strides(shape) if stride is None else stride
        return Tensor._over(data, shape, st, 0, dtype, Device.CUDA, True, keepalive)

    # -- access ---------------------------------------------------------------------------
    def raw(self) -> c_void_p:
        return self._view

    @property
    def shape(self):
        return self._shape

    @property
    def dtype(self) -> int:
        return self._dtype

    @property
    def device(self) -> int:
        return self._device

    def view_as(self, shape, stride, offset=0) -> "Tensor":
        """Another view of the same storage (shares it; this tensor must outlive the result)."""
        return Tensor._over(self._data, shape, stride, offset, self._dtype, self._device, False, self)

    def numpy(self) -> np.ndarray:
        """Copies to the host; 16-bit floats and codes come back as raw uint16 / uint8."""
        np_dtype = {1: np.uint8, 2: np.uint16, 4: np.float32 if self._dtype == DType.FLOAT else np.int32,
                    8: np.int64}[DTYPE_SIZE[self._dtype]]
        out = np.empty(self._shape, dtype=np_dtype)
        if out.size == 0:
            return out
        if self._device == Device.CPU:
            p = c_void_p()
            check(lib().fl_tensor_data_get_host_ptr(self._data, byref(p)))
            ctypes.memmove(out.ctypes.data, p.value, out.nbytes)
            return out
        host_data = c_void_p()
        check(lib().fl_tensor_data_borrow(out.ctypes.data_as(c_void_p), self._dtype, out.size, byref(host_data)))
        host = Tensor._over(host_data, out.shape, _contiguous_strides(out.shape), 0, self._dtype, Device.CPU, True, out)
        check(lib().fl_transfer(operators(), self.raw(), host.raw()))
        return out

    def __del__(self):
        try:
            L = _lib
            if L is None:
                return
            if self._view:
                L.fl_tensor_view_destroy(self._view)
                self._view = None
            if self._owns and self._data:
                L.fl_tensor_data_destroy(self._data)
                self._data = None
        except Exception:
            pass


class Transfer:
    """A copy that is still on its way (fl_transfer_t, flint/capi.h:71-73)."""

    def __init__(self, handle: c_void_p, keepalive=None):
        self._handle = handle
        self._keepalive = keepalive

    def wait(self) -> None:
        """Orders the compute stream's later work behind the copy; the caller does not stop."""
        check(lib().fl_transfer_wait(self._handle))

    def wait_sync(self) -> None:
        """Returns once the copy has finished."""
        check(lib().fl_transfer_wait_sync(self._handle))

    def __del__(self):
        try:
            if _lib is not None and self._handle:
                _lib.fl_transfer_destroy(self._handle)
                self._handle = None
        except Exception:
            pass


def transfer_async(src: Tensor):
    """fl_transfer_async (flint/capi.h:256-264): starts the upload of a page-locked host tensor and
    returns (device tensor of the same shape, Transfer); wait on the transfer before using the tensor."""
    data, handle = c_void_p(), c_void_p()
    check(lib().fl_transfer_async(src.raw(), Device.CUDA, byref(data), byref(handle)))
    dev = Tensor._over(data, src.shape, _contiguous_strides(src.shape), 0, src.dtype, Device.CUDA, True)
    return dev, Transfer(handle, keepalive=src)


def transfer_to_host_async(src: Tensor, dest: Tensor) -> Transfer:
    """Starts the download of a contiguous device tensor into a page-locked host tensor behind the
    work queued so far; `wait_sync()` on the result is when the host may read `dest`."""
    handle = c_void_p()
    check(lib().fl_sm100_transfer_to_host_async(src.raw(), dest.raw(), byref(handle)))
    return Transfer(handle, keepalive=(src, dest))


def copy(src: Tensor, dest: Tensor) -> Tensor:
    check(lib().fl_copy(operators(), src.raw(), dest.raw()))
    return dest


def cast(x: Tensor, dtype: int, out: Optional[Tensor] = None) -> Tensor:
    """fl_cast (flint/capi.h:249) between FLOAT, FLOAT16 and BFLOAT16."""
    if out is None:
        out = Tensor.empty(tuple(x.shape), dtype)
    check(lib().fl_cast(operators(), x.raw(), out.raw()))
    return out


def fill(t: Tensor, value: float) -> Tensor:
    check(lib().fl_fill(operators(), t.raw(), float(value)))
    return t


def add(a: Tensor, b: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """fl_add (flint/capi.h:483); `b` is expanded to `a`'s shape as a view first, as the Rust wrapper
    does (waifu/src/flint/functional.rs:80-108)."""
    if out is None:
        out = Tensor.empty(tuple(a.shape), a.dtype)
    bb = b if tuple(b.shape) == tuple(a.shape) else _broadcast_to(b, a)
    check(lib().fl_add(operators(), a.raw(), bb.raw(), out.raw()))
    return out


def _fp8_result(a: Tensor, rows: int) -> Tensor:
    """waifu/src/flint/functional.rs:655-662: (..., rows) in the activation's type on the device."""
    if len(a.shape) < 1:
        raise FlintError(FL_ERROR_INVALID_ARG, "fp8 matmul: an operand has no dimensions")
    return Tensor.empty(tuple(a.shape[:-1]) + (rows,), a.dtype, Device.CUDA)


def _broadcast_to(addend: Tensor, out: Tensor) -> Tensor:
    """waifu/src/flint/functional.rs:80-108: the addend expanded to out's shape as a zero-stride view."""
    ashape = addend.shape
    oshape = out.shape
    if len(ashape) > len(oshape):
        raise FlintError(FL_ERROR_INVALID_ARG, "fp8_matmul_add: the addend has more dimensions than the product")
    base = _contiguous_strides(ashape)
    shape, stride = [], []
    pad = len(oshape) - len(ashape)
    for i, o in enumerate(oshape):
        if i < pad:
            shape.append(o); stride.append(0)
            continue
        a = ashape[i - pad]
        if a == o:
            shape.append(o); stride.append(base[i - pad])
        elif a == 1:
            shape.append(o); stride.append(0)
        else:
            raise FlintError(FL_ERROR_INVALID_ARG, f"fp8_matmul_add: {ashape} does not broadcast to {oshape}")
    return addend.view_as(shape, stride, 0)


def linear_16(a: Tensor, weight: Tensor, addend: Optional[Tensor] = None) -> Tensor:
    """An unquantised linear layer as the reference's graph spells it (waifu/src/layers.rs:230-246):
    matmul (or matmul_add) of `a` (..., k) by the transposed view of `weight` (n, k)."""
    n, k = weight.shape
    wt = weight.view_as((k, n), (1, k), 0)
    out = Tensor.empty(tuple(a.shape[:-1]) + (n,), a.dtype, Device.CUDA)
    if addend is None:
        check(lib().fl_matmul(operators(), a.raw(), wt.raw(), out.raw()))
    else:
        ad = _broadcast_to(addend, out)  # held in a name: the view has to outlive the call
        check(lib().fl_matmul_add(operators(), a.raw(), wt.raw(), ad.raw(), out.raw()))
    return out


def fp8_matmul(a: Tensor, weight: Tensor, scale: Tensor) -> Tensor:
    """`a` (..., k) times the transpose of an FP8 weight (rows, k) with one <float> scale, as
    (..., rows); the activation is not narrowed (functional.rs:664-680)."""
    out = _fp8_result(a, weight.shape[0])
    check(lib().fl_fp8_matmul(a.raw(), weight.raw(), scale.raw(), out.raw()))
    return out


def fp8_matmul_add(a: Tensor, weight: Tensor, scale: Tensor, addend: Tensor, expand: bool = True) -> Tensor:
    """fp8_matmul plus a bias or residual added in the epilogue, one rounding (functional.rs:682-703).
    `expand` pre-broadcasts the addend to the product's shape as a view, as the Rust wrapper does;
    pass False to hand the addend over as it is, as the reference's C++ tests do."""
    out = _fp8_result(a, weight.shape[0])
    if addend.dtype != out.dtype:
        raise FlintError(FL_ERROR_INVALID_ARG, "fp8_matmul_add: the addend is not of the product's type")
    ad = _broadcast_to(addend, out) if expand else addend
    check(lib().fl_fp8_matmul_add(a.raw(), weight.raw(), scale.raw(), ad.raw(), out.raw()))
    return out


def fp8_linear(a: Tensor, weight: Tensor, scales: Tensor, bias: Optional[Tensor] = None,
               residual: Optional[Tensor] = None, act: int = ACT_NONE, out: Optional[Tensor] = None) -> Tensor:
    """Dynamic per-token e4m3 activation x e4m3 weight with per-channel (or per-tensor) scales and
    the fused bias / GELU-tanh / residual epilogue."""
    if out is None:
        out = _fp8_result(a, weight.shape[0])
    check(lib().fl_fp8_linear(a.raw(), weight.raw(), scales.raw(), bias.raw() if bias else None,
                              residual.raw() if residual else None, int(act), out.raw()))
    return out


def fp8_linear_static(a: Tensor, weight: Tensor, scales: Tensor, bias: Optional[Tensor] = None,
                      residual: Optional[Tensor] = None, act: int = ACT_NONE, out: Optional[Tensor] = None) -> Tensor:
    """fp8_linear through the entry point that allocates nothing: its activation scratch is a fixed
    16.3 MiB device array inside the library (at most 65536 rows and 16 Mi elements of m * k).
    For hosts that run with the whole card budgeted or cannot take an allocation's device-wide
    stall mid-pass. `out` should be passed by such a host; when it is None it is allocated here,
    by this wrapper, which is a convenience of the wrapper and not of the entry point."""
    if out is None:
        out = _fp8_result(a, weight.shape[0])
    check(lib().fl_fp8_linear_static(a.raw(), weight.raw(), scales.raw(), bias.raw() if bias else None,
                                     residual.raw() if residual else None, int(act), out.raw()))
    return out


def fp8_linear_scatter(a: Tensor, weight: Tensor, scales: Tensor, dests: Sequence[Tensor], col0: int,
                       bias: Optional[Tensor] = None, residual: Optional[Tensor] = None, act: int = ACT_NONE) -> None:
    """fp8_linear whose result is written by the epilogue into columns [col0, col0 + rows) of every
    matrix in `dests` (this GPU's and its peers'): the fused all-gather of an output-channel split."""
    arr = (c_void_p * len(dests))(*[d.raw() for d in dests])
    check(lib().fl_fp8_linear_scatter(a.raw(), weight.raw(), scales.raw(), bias.raw() if bias else None,
                                      residual.raw() if residual else None, int(act), arr, len(dests), int(col0)))


def fp8_linear_amax(a: Tensor, weight: Tensor, scales: Tensor, row_amax: Tensor, bias: Optional[Tensor] = None,
                    residual: Optional[Tensor] = None, act: int = ACT_NONE, out: Optional[Tensor] = None) -> Tensor:
    """fp8_linear that also leaves each output row's largest magnitude (as rounded) in `row_amax`."""
    if out is None:
        out = _fp8_result(a, weight.shape[0])
    check(lib().fl_fp8_linear_amax(a.raw(), weight.raw(), scales.raw(), bias.raw() if bias else None,
                                   residual.raw() if residual else None, int(act), out.raw(), row_amax.raw()))
    return out


def fp8_row_amax(x: Tensor, row_amax: Optional[Tensor] = None) -> Tensor:
    """The largest magnitude of each row of a 16-bit matrix (its rows may be a wider matrix's)."""
    if row_amax is None:
        row_amax = Tensor.empty((x.shape[0],), DType.FLOAT)
    check(lib().fl_fp8_row_amax(x.raw(), row_amax.raw()))
    return row_amax


def fp8_quantize_scatter(x: Tensor, row_amax: Tensor, dests: Sequence[Tensor], col0: int,
                         row_scales: Optional[Tensor] = None) -> None:
    """Per-row e4m3 of `x` with the rows' maxima given, the codes written into columns
    [col0, col0 + k) of every matrix in `dests` (this GPU's and its peers')."""
    arr = (c_void_p * len(dests))(*[d.raw() for d in dests])
    check(lib().fl_fp8_quantize_scatter(x.raw(), row_amax.raw(), arr, len(dests), int(col0),
                                        row_scales.raw() if row_scales else None))


def fp8_linear_quantized_scatter(codes: Tensor, row_scales: Tensor, weight: Tensor, scales: Tensor, dests: Sequence[Tensor],
                                 col0: int, bias: Optional[Tensor] = None, residual: Optional[Tensor] = None,
                                 act: int = ACT_NONE) -> None:
    """fp8_linear_quantized whose result lands in columns [col0, col0 + rows) of every matrix in `dests`."""
    arr = (c_void_p * len(dests))(*[d.raw() for d in dests])
    check(lib().fl_fp8_linear_quantized_scatter(codes.raw(), row_scales.raw(), weight.raw(), scales.raw(),
                                                bias.raw() if bias else None, residual.raw() if residual else None,
                                                int(act), arr, len(dests), int(col0)))


PEER_HEADER = 64


class PeerGroup:
    """The mailboxes of fl_sm100_peer_exchange for the ranks of one box and the epoch they count.

    `exchange_handles(handle) -> list of every rank's handle` is the caller's way of passing 64-byte
    handles between the processes (an all_gather_object, a file, a pipe)."""

    def __init__(self, rank: int, world: int, capacity: int, exchange_handles):
        self.rank, self.world = rank, world
        width = PEER_HEADER + max(int(capacity), 0)
        rows = max(world, -(-(2 << 20) // (4 * width)))  # storage of its own starts at 2 MiB
        self._own = Tensor.empty((rows, width), DType.INT32, hint=AllocHint.WEIGHT)
        copy(Tensor.from_numpy(np.zeros((rows, width), np.int32), DType.INT32), self._own)
        synchronize()
        handles = exchange_handles(ipc_export(self._own))
        self._peers = {r: ipc_import(handles[r], (rows, width), DType.INT32) for r in range(world) if r != rank}
        self._boxes = [(self._own if r == rank else self._peers[r]).view_as((world, width), (width, 1)) for r in range(world)]
        self._arr = (c_void_p * world)(*[b.raw() for b in self._boxes])
        self.epoch = 0

    def exchange(self, row_amax: Optional[Tensor] = None, max_polls: int = 0) -> None:
        """A barrier on the stream among the ranks; with `row_amax`, also its maximum over the ranks."""
        self.epoch += 1
        check(lib().fl_sm100_peer_exchange(self._arr, self.world, self.rank, self.epoch,
                                           row_amax.raw() if row_amax else None, int(max_polls)))


def ipc_export(t: Tensor) -> bytes:
    """The 64-byte handle of a device tensor made by Tensor.empty(..., hint=AllocHint.WEIGHT) of
    2 MiB or more, for a peer process."""
    buf = ctypes.create_string_buffer(64)
    check(lib().fl_sm100_ipc_export(t._data, buf))
    return bytes(buf.raw)


def ipc_import(handle: bytes, shape: Sequence[int], dtype: int) -> Tensor:
    """Maps a peer process's device tensor (same box) from its handle."""
    numel = int(np.prod(shape))
    data = c_void_p()
    buf = ctypes.create_string_buffer(handle, 64)
    check(lib().fl_sm100_ipc_import(buf, dtype, max(numel, 1), byref(data)))
    return Tensor._over(data, shape, _contiguous_strides(shape), 0, dtype, Device.CUDA, True)


def nvfp4_linear(a: Tensor, codes: Tensor, block_scales: Tensor, global_scale: Tensor,
                 bias: Optional[Tensor] = None, residual: Optional[Tensor] = None, act: int = ACT_NONE,
                 out: Optional[Tensor] = None) -> Tensor:
    """Dynamic per-16-block e2m1 activation x NVFP4 weight with the same fused epilogue."""
    if out is None:
        out = _fp8_result(a, codes.shape[0])
    check(lib().fl_nvfp4_linear(a.raw(), codes.raw(), block_scales.raw(), global_scale.raw(),
                                bias.raw() if bias else None, residual.raw() if residual else None, int(act),
                                out.raw()))
    return out


def quantize_fp8_rows(w: Tensor):
    rows, k = w.shape
    codes = Tensor.empty((rows, k), DType.FP8E4M3)
    scales = Tensor.empty((rows,), DType.FLOAT)
    check(lib().fl_quantize_fp8_rows(w.raw(), codes.raw(), scales.raw()))
    return codes, scales


def fp8_layernorm_quantize(x: Tensor, scale: Optional[Tensor] = None, shift: Optional[Tensor] = None,
                           eps: float = 1e-6, codes: Optional[Tensor] = None, row_scales: Optional[Tensor] = None):
    """Layer norm over the last dimension, adaLN modulation n * scale + n + shift, narrowing to x's
    type and per-row e4m3 quantisation in one pass; returns (codes, row_scales)."""
    rows = 1
    for d in x.shape[:-1]:
        rows *= d
    if codes is None:
        codes = Tensor.empty(tuple(x.shape), DType.FP8E4M3)
    if row_scales is None:
        row_scales = Tensor.empty((rows,), DType.FLOAT)
    check(lib().fl_fp8_layernorm_quantize(x.raw(), scale.raw() if scale else None, shift.raw() if shift else None,
                                          float(eps), codes.raw(), row_scales.raw()))
    return codes, row_scales


def fp8_swiglu_quantize(x: Tensor, codes: Optional[Tensor] = None, row_scales: Optional[Tensor] = None):
    """silu(gate) * value over the two halves of the last dimension, narrowed to x's type, then
    per-row e4m3 in the same pass; returns (codes, row_scales)."""
    rows = 1
    for d in x.shape[:-1]:
        rows *= d
    if codes is None:
        codes = Tensor.empty(tuple(x.shape[:-1]) + (x.shape[-1] // 2,), DType.FP8E4M3)
    if row_scales is None:
        row_scales = Tensor.empty((rows,), DType.FLOAT)
    check(lib().fl_fp8_swiglu_quantize(x.raw(), codes.raw(), row_scales.raw()))
    return codes, row_scales


def fp8_linear_quantized_grouped(codes: Tensor, row_scales: Tensor, weight: Tensor, scales: Tensor, bias: Optional[Tensor],
                                 residual: Optional[Tensor], act: int, rows_per_group: int, out: Tensor) -> Tensor:
    """fp8_linear_quantized whose rows come in groups of `rows_per_group` (a multiple of 256), each
    with its own row of `scales` (groups, n) and `bias` (groups, n)."""
    check(lib().fl_fp8_linear_quantized_grouped(codes.raw(), row_scales.raw(), weight.raw(), scales.raw(),
                                                bias.raw() if bias else None, residual.raw() if residual else None,
                                                int(act), int(rows_per_group), out.raw()))
    return out


def fp8_linear_quantized(codes: Tensor, row_scales: Tensor, weight: Tensor, scales: Tensor, bias: Optional[Tensor],
                         residual: Optional[Tensor], act: int, out: Tensor) -> Tensor:
    """fp8_linear for an activation that is e4m3 codes with per-row scales already."""
    check(lib().fl_fp8_linear_quantized(codes.raw(), row_scales.raw(), weight.raw(), scales.raw(),
                                        bias.raw() if bias else None, residual.raw() if residual else None, int(act),
                                        out.raw()))
    return out


def qk_norm_rope(qkv: Tensor, cos: Tensor, sin: Tensor, heads: int, eps: float = 1e-6,
                 q_weight: Optional[Tensor] = None, k_weight: Optional[Tensor] = None) -> Tensor:
    """In place on a fused projection's output (..., 3 * heads * head_dim): per-head RMS norm of the
    q and k thirds and the rotation of their even/odd pairs; returns qkv."""
    check(lib().fl_qk_norm_rope(qkv.raw(), q_weight.raw() if q_weight else None, k_weight.raw() if k_weight else None,
                                cos.raw(), sin.raw(), float(eps), int(heads)))
    return qkv


class MaskType:
    """fl_mask_type_t (flint/capi.h:118-133)."""
    NONE = 0
    CAUSAL = 1
    BLOCK_CAUSAL = 2
    BLOCK_DIAGONAL = 3


def attention(q: Tensor, k: Tensor, v: Tensor, mask_type: int = MaskType.NONE, block_size: int = 0,
              out: Optional[Tensor] = None) -> Tensor:
    """fl_attention (flint/capi.h:532-544): q (N, heads, L, D), k and v (N, kv_heads, S, D), any
    strides with a contiguous last dimension; out (N, heads, L, D), contiguous when made here."""
    if out is None:
        out = Tensor.empty(tuple(q.shape), q.dtype)
    check(lib().fl_attention(operators(), q.raw(), k.raw(), v.raw(), int(mask_type), int(block_size), out.raw()))
    return out


def quantize_fp8_activation(a: Tensor):
    m, k = a.shape
    codes = Tensor.empty((m, k), DType.FP8E4M3)
    scales = Tensor.empty((m,), DType.FLOAT)
    check(lib().fl_quantize_fp8_activation(a.raw(), codes.raw(), scales.raw()))
    return codes, scales


def quantize_nvfp4(w: Tensor):
    rows, k = w.shape
    codes = Tensor.empty((rows, k // 2), DType.FP4E2M1X2)
    sf = Tensor.empty((rows, k // 16), DType.FP8E4M3)
    g = Tensor.empty((1,), DType.FLOAT)
    check(lib().fl_quantize_nvfp4(w.raw(), codes.raw(), sf.raw(), g.raw()))
    return codes, sf, g
