"""fl_matmul / fl_matmul_add for the unquantised linear layer (16-bit operands, fp32
accumulation, one rounding) against the oracle's float32 product of the widened operands."""
import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("is_bf16", [False, True])
@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (17, 128, 64), (129, 264, 96), (300, 200, 256), (600, 512, 1024)])
def test_linear_16(flint, oracle, is_bf16, m, n, k):
    F = flint
    rng = np.random.default_rng(m * 7 + n + k)
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    a = oracle.narrow(randn(rng, (m, k)), is_bf16)
    w = oracle.narrow(randn(rng, (n, k), 0.05), is_bf16)
    bias = oracle.narrow(randn(rng, (n,), 0.1), is_bf16)
    dev = lambda x: F.Tensor.from_numpy(x, dt, F.Device.CUDA)
    acc = oracle.gemm_f32_nt(oracle.widen(a, is_bf16), oracle.widen(w, is_bf16))
    got = F.linear_16(dev(a), dev(w)).numpy()
    check_parity(oracle, got, oracle.epilogue(acc, out_is_bf16=is_bf16), is_bf16, what="matmul")
    got_b = F.linear_16(dev(a), dev(w), dev(bias)).numpy()
    check_parity(oracle, got_b, oracle.epilogue(acc, bias=bias, out_is_bf16=is_bf16), is_bf16, what="matmul_add")


def test_other_layouts_are_refused(flint):
    F = flint
    a = F.Tensor.empty((4, 16), F.DType.FLOAT16)
    b = F.Tensor.empty((16, 8), F.DType.FLOAT16)  # row-major (k, n): not the transposed-weight view
    out = F.Tensor.empty((4, 8), F.DType.FLOAT16)
    code = F.lib().fl_matmul(F.operators(), a.raw(), b.raw(), out.raw())
    assert code == F.FL_ERROR_INVALID_ARG and b"not implemented" in F.lib().fl_get_last_error_message()
    f32 = F.Tensor.empty((4, 16), F.DType.FLOAT)
    assert F.lib().fl_matmul(F.operators(), f32.raw(), b.raw(), out.raw()) == F.FL_ERROR_INVALID_ARG


@pytest.mark.parametrize("is_bf16", [False, True])
@pytest.mark.parametrize("m,n,k", [(1, 3072, 3072), (2, 264, 72), (16, 1184, 4104), (9, 72, 12288), (5, 8, 16), (1, 16384, 2048)])
def test_few_rows(flint, oracle, is_bf16, m, n, k):
    """At most 16 rows take the one-launch bandwidth-shaped kernel (the reference's GEMV case,
    flint/cuda/matvec.cu): plain, with a bias, and with a residual of out's shape."""
    F = flint
    rng = np.random.default_rng(m * 11 + n + k)
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    a = oracle.narrow(randn(rng, (m, k)), is_bf16)
    w = oracle.narrow(randn(rng, (n, k), 0.05), is_bf16)
    bias = oracle.narrow(randn(rng, (n,), 0.1), is_bf16)
    res = oracle.narrow(randn(rng, (m, n)), is_bf16)
    dev = lambda x: F.Tensor.from_numpy(x, dt, F.Device.CUDA)
    acc = oracle.gemm_f32_nt(oracle.widen(a, is_bf16), oracle.widen(w, is_bf16))
    check_parity(oracle, F.linear_16(dev(a), dev(w)).numpy(), oracle.epilogue(acc, out_is_bf16=is_bf16), is_bf16, what="few rows")
    check_parity(oracle, F.linear_16(dev(a), dev(w), dev(bias)).numpy(), oracle.epilogue(acc, bias=bias, out_is_bf16=is_bf16),
                 is_bf16, what="few rows + bias")
    check_parity(oracle, F.linear_16(dev(a), dev(w), dev(res)).numpy(), oracle.epilogue(acc, residual=res, out_is_bf16=is_bf16),
                 is_bf16, what="few rows + residual")
