"""The C-ABI library without a GPU: it loads, exports every symbol include/flint_sm100.h
declares, and refuses bad arguments with the reference's codes (flint/capi_test.cc:448-487,
waifu/tests/tensor.rs:142-155). No compute call is made here."""
import ctypes
import os
import re
from ctypes import byref, c_int32, c_void_p

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "flint_sm100.h")).read()
    return sorted(set(re.findall(r"FLAPI\s+[\w\s\*]+?\b(fl_\w+)\s*\(", text)))


def test_header_declares_the_reference_signatures():
    names = declared_symbols()
    for must in ("fl_init", "fl_get_last_error_code", "fl_get_last_error_message", "fl_operators_create",
                 "fl_operators_destroy", "fl_tensor_data_create", "fl_tensor_data_borrow", "fl_tensor_data_destroy",
                 "fl_tensor_data_get_host_ptr", "fl_tensor_view_create", "fl_tensor_view_destroy", "fl_transfer",
                 "fl_fp8_available", "fl_fp8_matmul", "fl_fp8_matmul_add", "fl_fp8_linear", "fl_nvfp4_linear"):
        assert must in names


def test_library_exports_every_declared_symbol(flint):
    L = flint.lib()
    for name in declared_symbols():
        assert hasattr(L, name), f"{name} is declared in the header but not exported"


def test_enum_values_are_the_reference_ones(flint):
    # flint/capi.h:84-106
    assert (flint.DType.FLOAT, flint.DType.FLOAT16, flint.DType.FP8E4M3) == (1, 4, 10)
    assert (flint.Device.CPU, flint.Device.CUDA, flint.Device.CUDA_HOST, flint.Device.UNKNOWN) == (0, 1, 2, 5)
    assert (flint.FL_ERROR_INVALID_ARG, flint.FL_ERROR_ABORTED, flint.FL_ERROR_OUT_OF_MEMORY) == (0x100, 0x102, 0x103)


def test_availability_never_errors_for_a_device_without_kernels(flint):
    # flint/capi.cc:962-975,1039-1045: CPU, Metal and Vulkan answer 0, not an error.
    L = flint.lib()
    for dev in (flint.Device.CPU, flint.Device.CUDA_HOST, flint.Device.METAL, flint.Device.VULKAN):
        out = c_int32(7)
        assert L.fl_fp8_available(dev, byref(out)) == 0
        assert out.value == 0
    assert L.fl_fp8_available(flint.Device.CPU, None) == flint.FL_ERROR_INVALID_ARG
    assert b"out is null" in L.fl_get_last_error_message()
    assert L.fl_get_last_error_code() == flint.FL_ERROR_INVALID_ARG
    out = c_int32(0)
    assert L.fl_fp8_available(flint.Device.CPU, byref(out)) == 0
    assert L.fl_get_last_error_code() == 0 and L.fl_get_last_error_message() == b""


def cpu(flint, arr, dtype):
    return flint.Tensor.from_numpy(arr, dtype, flint.Device.CPU)


def test_cpu_operands_are_refused_with_the_reference_message(flint):
    # waifu/tests/tensor.rs:142-155 / flint/capi.cc:1095
    a = cpu(flint, np.zeros((2, 32), np.uint16), flint.DType.FLOAT16)
    w = cpu(flint, np.zeros((8, 32), np.uint8), flint.DType.FP8E4M3)
    s = cpu(flint, np.ones(1, np.float32), flint.DType.FLOAT)
    out = cpu(flint, np.zeros((2, 8), np.uint16), flint.DType.FLOAT16)
    L = flint.lib()
    assert L.fl_fp8_matmul(a.raw(), w.raw(), s.raw(), out.raw()) == flint.FL_ERROR_INVALID_ARG
    assert b"no FP8 kernels" in L.fl_get_last_error_message()


def test_argument_refusals(flint):
    # flint/capi_test.cc:468-486 and flint/capi.cc:979-1035: all INVALID_ARG, checked before any device work.
    L = flint.lib()
    F = flint
    a = cpu(F, np.zeros((2, 32), np.uint16), F.DType.FLOAT16)
    w = cpu(F, np.zeros((8, 32), np.uint8), F.DType.FP8E4M3)
    s = cpu(F, np.ones(1, np.float32), F.DType.FLOAT)
    out = cpu(F, np.zeros((2, 8), np.uint16), F.DType.FLOAT16)

    def refused(*views, fn=L.fl_fp8_matmul, needle=None):
        code = fn(*[v.raw() if v is not None else None for v in views])
        assert code == F.FL_ERROR_INVALID_ARG, L.fl_get_last_error_message()
        if needle:
            assert needle in L.fl_get_last_error_message(), L.fl_get_last_error_message()

    # the weight is not fp8
    refused(a, cpu(F, np.zeros((8, 32), np.uint8), F.DType.UINT8), s, out, needle=b"not <fp8e4m3>")
    # a scale per row
    refused(a, w, cpu(F, np.ones(8, np.float32), F.DType.FLOAT), out, needle=b"single <float>")
    # a weight of three dimensions
    refused(a, cpu(F, np.zeros((2, 4, 32), np.uint8), F.DType.FP8E4M3), s, out, needle=b"(rows, k)")
    # the left operand is float32
    refused(cpu(F, np.zeros((2, 32), np.float32), F.DType.FLOAT), w, s, out, needle=b"not <float16>")
    # fewer than two dimensions
    refused(cpu(F, np.zeros((32,), np.uint16), F.DType.FLOAT16), w, s, out, needle=b"fewer than two")
    # k disagrees
    refused(cpu(F, np.zeros((2, 16), np.uint16), F.DType.FLOAT16), w, s, out, needle=b"disagree about k")
    # out of the wrong shape / dtype
    refused(a, w, s, cpu(F, np.zeros((2, 16), np.uint16), F.DType.FLOAT16), needle=b"was expected")
    refused(a, w, s, cpu(F, np.zeros((2, 8), np.float32), F.DType.FLOAT), needle=b"out is not")
    # a non-contiguous left operand
    big = cpu(F, np.zeros((2, 64), np.uint16), F.DType.FLOAT16)
    refused(big.view_as((2, 32), (64, 1)), w, s, out, needle=b"not contiguous")
    # an addend of the wrong type, and one with more dimensions than out
    refused(a, w, s, cpu(F, np.zeros(8, np.float32), F.DType.FLOAT), out, fn=L.fl_fp8_matmul_add, needle=b"addend")
    refused(a, w, s, cpu(F, np.zeros((1, 2, 8), np.uint16), F.DType.FLOAT16), out, fn=L.fl_fp8_matmul_add, needle=b"addend")
    # null views
    assert L.fl_fp8_matmul(None, w.raw(), s.raw(), out.raw()) == F.FL_ERROR_INVALID_ARG


def test_view_bounds_are_checked_at_creation(flint):
    # flint/capi.h:217-231
    L = flint.lib()
    data = c_void_p()
    buf = np.zeros(16, np.float32)
    assert L.fl_tensor_data_borrow(buf.ctypes.data_as(c_void_p), 1, 16, byref(data)) == 0
    view = c_void_p()
    sh = (c_int32 * 2)(4, 4)
    st = (c_int32 * 2)(4, 1)
    assert L.fl_tensor_view_create(data, sh, st, 2, 0, byref(view)) == 0
    L.fl_tensor_view_destroy(view)
    assert L.fl_tensor_view_create(data, sh, st, 2, 1, byref(view)) == flint.FL_ERROR_INVALID_ARG
    assert b"reaches element 16" in L.fl_get_last_error_message()
    st0 = (c_int32 * 2)(0, 1)  # a zero stride repeats rows and is allowed
    assert L.fl_tensor_view_create(data, sh, st0, 2, 12, byref(view)) == 0
    L.fl_tensor_view_destroy(view)
    neg = (c_int32 * 2)(4, -1)
    assert L.fl_tensor_view_create(data, sh, neg, 2, 0, byref(view)) == flint.FL_ERROR_INVALID_ARG
    L.fl_tensor_data_destroy(data)
    # misaligned borrowed bytes are refused (flint/capi.cc:386-394)
    raw = np.zeros(9, np.uint8)
    addr = raw.ctypes.data + (1 if raw.ctypes.data % 2 == 0 else 0)
    assert L.fl_tensor_data_borrow(c_void_p(addr), 4, 2, byref(data)) == flint.FL_ERROR_INVALID_ARG


def test_host_pointer_of_host_storage(flint):
    L = flint.lib()
    data = c_void_p()
    assert L.fl_tensor_data_create(flint.Device.CPU, flint.DType.FLOAT, 8, 0, byref(data)) == 0
    p = c_void_p()
    assert L.fl_tensor_data_get_host_ptr(data, byref(p)) == 0 and p.value
    L.fl_tensor_data_destroy(data)
    assert L.fl_tensor_data_create(flint.Device.CPU, flint.DType.FLOAT, 0, 0, byref(data)) == flint.FL_ERROR_INVALID_ARG


def test_no_gpu_means_a_loud_failure_not_a_fallback(flint):
    """Without a B200 the operators cannot be created and device storage cannot be had: the
    product path has no CPU route."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = flint.lib()
    h = c_void_p()
    assert L.fl_operators_create(flint.Device.CUDA, byref(h)) == flint.FL_ERROR_ABORTED
    assert L.fl_operators_create(flint.Device.CPU, byref(h)) == flint.FL_ERROR_INVALID_ARG
    assert not flint.fp8_available(flint.Device.CUDA)
    with pytest.raises(flint.FlintError):
        flint.Tensor.empty((2, 2), flint.DType.FLOAT16, flint.Device.CUDA)


def _prototypes(text):
    """name -> 'return-type name(parameters)' with whitespace squeezed, of every FLAPI declaration."""
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    out = {}
    for m in re.finditer(r"FLAPI\s+([^;{]+?\b(fl_\w+)\s*\([^;{]*?\))\s*;", text, flags=re.S):
        proto = re.sub(r"\s+", " ", m.group(1)).strip()
        proto = re.sub(r"\(\s+", "(", proto)
        proto = re.sub(r"\s+\)", ")", proto)
        proto = re.sub(r",\s*\)", ")", proto)
        out[m.group(2)] = proto
    return out


def test_part_one_prototypes_equal_the_reference_headers(oracle):
    """Every declaration of the header's first part is, token for token, the declaration of the same
    name in the reference's flint/capi.h (return type, parameter types and parameter names)."""
    ref_dir = oracle.reference_dir()
    if not ref_dir:
        pytest.skip("no reference checkout here")
    ours_text = open(os.path.join(ROOT, "include", "flint_sm100.h")).read()
    part1 = ours_text.split("Part 2: additive entry points")[0]
    ours = _prototypes(part1)
    theirs = _prototypes(open(os.path.join(ref_dir, "flint", "capi.h")).read())
    assert len(ours) >= 25
    for name, proto in ours.items():
        assert name in theirs, f"{name} is in part 1 but the reference does not declare it"
        assert proto == theirs[name], f"{name}:\n  ours      {proto}\n  reference {theirs[name]}"
    # the part-1 enum values, against the reference's own enumerators
    ref_text = open(os.path.join(ref_dir, "flint", "capi.h")).read()
    for enumerator in re.findall(r"\b(FL_(?:DTYPE|DEVICE|ALLOC|MASK)_\w+)\s*=\s*(\d+)", part1):
        m = re.search(r"\b%s\s*=\s*(\d+)" % enumerator[0], ref_text)
        if m:  # the two additive dtypes have no counterpart
            assert m.group(1) == enumerator[1], enumerator
    for code in re.findall(r"#define\s+(FL_\w+)\s+(\w+)", part1):
        m = re.search(r"#define\s+%s\s+(\w+)" % code[0], ref_text)
        if m:
            assert int(m.group(1), 0) == int(code[1], 0), code


def test_storage_bound_is_the_reference_one(flint):
    # flint/tensor.h:41: storage holds at most 2^30 elements; refused before anything is allocated
    L = flint.lib()
    data = c_void_p()
    assert L.fl_tensor_data_create(flint.Device.CPU, flint.DType.UINT8, (1 << 30) + 1, 0, byref(data)) == flint.FL_ERROR_INVALID_ARG
    assert b"too many elements" in L.fl_get_last_error_message()
    assert L.fl_tensor_data_create(flint.Device.CPU, flint.DType.UINT8, 16, 9, byref(data)) == flint.FL_ERROR_INVALID_ARG


def test_asynchronous_copy_refuses_every_direction_but_its_own(flint):
    # flint/cuda/to_device.cc:143-160: page-locked host memory to the GPU, nothing else
    F, L = flint, flint.lib()
    src = cpu(F, np.zeros((4, 4), np.float32), F.DType.FLOAT)
    dest, handle = c_void_p(), c_void_p()
    assert L.fl_transfer_async(src.raw(), F.Device.CUDA, byref(dest), byref(handle)) == F.FL_ERROR_INVALID_ARG
    assert b"from cuda-host to cuda, not from cpu to cuda" in L.fl_get_last_error_message()
    assert L.fl_transfer_async(src.raw(), F.Device.CUDA, None, byref(handle)) == F.FL_ERROR_INVALID_ARG
    assert L.fl_transfer_wait(None) == F.FL_ERROR_INVALID_ARG
    L.fl_transfer_destroy(None)
    # the elementwise operators want every view on the operators' device
    assert L.fl_add(None, src.raw(), src.raw(), src.raw()) == F.FL_ERROR_INVALID_ARG
    assert L.fl_cast(c_void_p(1), src.raw(), src.raw()) == F.FL_ERROR_INVALID_ARG
    assert b"not on the operators' device" in L.fl_get_last_error_message()


def test_row_group_refusals(flint):
    """fl_fp8_linear_quantized_grouped checks its groups before any device work: a group size that is
    no multiple of 256, scales and bias that are not one row per group."""
    F = flint
    L = F.lib()
    m, n, k, rpg = 512, 8, 32, 256
    codes = cpu(F, np.zeros((m, k), np.uint8), F.DType.FP8E4M3)
    rs = cpu(F, np.ones(m, np.float32), F.DType.FLOAT)
    w = cpu(F, np.zeros((n, k), np.uint8), F.DType.FP8E4M3)
    scales = cpu(F, np.ones((2, n), np.float32), F.DType.FLOAT)
    bias = cpu(F, np.zeros((2, n), np.uint16), F.DType.BFLOAT16)
    out = cpu(F, np.zeros((m, n), np.uint16), F.DType.BFLOAT16)

    def call(scales_v, bias_v, group_rows):
        return L.fl_fp8_linear_quantized_grouped(codes.raw(), rs.raw(), w.raw(), scales_v.raw(),
                                                 bias_v.raw() if bias_v is not None else None, None, 0, group_rows, out.raw())

    assert call(scales, bias, 100) == F.FL_ERROR_INVALID_ARG and b"multiple of 256" in L.fl_get_last_error_message()
    assert call(scales, bias, 0) == F.FL_ERROR_INVALID_ARG and b"multiple of 256" in L.fl_get_last_error_message()
    one_row = cpu(F, np.ones(n, np.float32), F.DType.FLOAT)
    assert call(one_row, bias, rpg) == F.FL_ERROR_INVALID_ARG and b"(groups, rows)" in L.fl_get_last_error_message()
    assert call(scales, cpu(F, np.zeros(n, np.uint16), F.DType.BFLOAT16), rpg) == F.FL_ERROR_INVALID_ARG
    assert b"(groups, rows)" in L.fl_get_last_error_message()
    # well-formed groups on CPU operands end where every FP8 entry point ends without a device
    assert call(scales, bias, rpg) == F.FL_ERROR_INVALID_ARG and b"no FP8 kernels" in L.fl_get_last_error_message()
