"""fl_matmul / fl_matmul_add: the unquantised linear layer (16-bit operands, fp32 accumulation, one
rounding) against the oracle's float32 product of the widened operands, and the other layouts the
reference's matmul takes (float32, batches, row-major right operands, odd extents) against float64."""
import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


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


@pytest.mark.parametrize("is_bf16", [False, True])
@pytest.mark.parametrize("m,n,k", [(5, 6144, 2048), (16, 3080, 2056), (33, 3072, 2048), (64, 16384, 2048), (2, 16392, 2304),
                                   (24, 19080, 2048)])
def test_few_rows_wide_weight(flint, oracle, is_bf16, m, n, k):
    """At most 64 rows against a wide 16-bit weight: the weight on the M side of the tensor-core
    instruction. No addend, a bias, a residual; a ragged last block of channels, rows whose bytes
    end inside a stage, more CTAs than SMs."""
    F = flint
    rng = np.random.default_rng(m * 11 + n + k)
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    a = oracle.narrow(randn(rng, (m, k)), is_bf16)
    w = oracle.narrow(randn(rng, (n, k), 0.05), is_bf16)
    bias = oracle.narrow(randn(rng, (n,), 0.1), is_bf16)
    res = oracle.narrow(randn(rng, (m, n)), is_bf16)
    dev = lambda x: F.Tensor.from_numpy(x, dt, F.Device.CUDA)
    acc = oracle.gemm_f32_nt(oracle.widen(a, is_bf16), oracle.widen(w, is_bf16))
    ad, wd = dev(a), dev(w)
    check_parity(oracle, F.linear_16(ad, wd).numpy(), oracle.epilogue(acc, out_is_bf16=is_bf16), is_bf16, what="matmul")
    check_parity(oracle, F.linear_16(ad, wd, dev(bias)).numpy(), oracle.epilogue(acc, bias=bias, out_is_bf16=is_bf16), is_bf16,
                 what="matmul_add bias")
    check_parity(oracle, F.linear_16(ad, wd, dev(res)).numpy(), oracle.epilogue(acc, residual=res, out_is_bf16=is_bf16), is_bf16,
                 what="matmul_add residual")


def matmul(F, a, b, out_dtype, addend=None):
    out = F.Tensor.empty(tuple(a.shape[:-1]) + (b.shape[-1],), out_dtype)
    if addend is None:
        F.check(F.lib().fl_matmul(F.operators(), a.raw(), b.raw(), out.raw()))
    else:
        ad = addend if tuple(addend.shape) == tuple(out.shape) else F._broadcast_to(addend, out)
        F.check(F.lib().fl_matmul_add(F.operators(), a.raw(), b.raw(), ad.raw(), out.raw()))
    return out


def test_float32_and_other_layouts(flint, oracle):
    """What the reference's matmul takes beyond the linear-layer case (flint/cuda/matmul.cc:315-343):
    float32 operands, a right operand that lies row-major, extents that are no multiples of 8 (the
    129-channel projection of waifu/src/qwen_image/dit.rs:374-381), a float32 result from half operands."""
    F = flint
    rng = np.random.default_rng(41)
    fl = F.DType.FLOAT
    for (m, n, k) in [(33, 20, 129), (200, 264, 96), (1, 7, 5)]:
        a = randn(rng, (m, k))
        b = randn(rng, (k, n), 0.1)
        bias = randn(rng, (n,))
        res = randn(rng, (m, n))
        want = a.astype(np.float64) @ b.astype(np.float64)
        got = matmul(F, dev(F, a, fl), dev(F, b, fl), fl).numpy()
        assert oracle.rel_l2(got, want) <= 1e-6
        got = matmul(F, dev(F, a, fl), dev(F, b, fl), fl, dev(F, bias, fl)).numpy()
        assert oracle.rel_l2(got, want + bias) <= 1e-6
        got = matmul(F, dev(F, a, fl), dev(F, b, fl), fl, dev(F, res, fl)).numpy()
        assert oracle.rel_l2(got, want + res) <= 1e-6
        # the same right operand handed over as the transposed view of an (n, k) weight
        bt = dev(F, np.ascontiguousarray(b.T), fl).view_as((k, n), (1, k))
        assert oracle.rel_l2(matmul(F, dev(F, a, fl), bt, fl).numpy(), want) <= 1e-6
        for is_bf16, dt in ((False, F.DType.FLOAT16), (True, F.DType.BFLOAT16)):
            a16, b16 = oracle.narrow(a, is_bf16), oracle.narrow(b, is_bf16)
            exact = oracle.widen(a16, is_bf16).astype(np.float64) @ oracle.widen(b16, is_bf16).astype(np.float64)
            got16 = matmul(F, dev(F, a16, dt), dev(F, b16, dt), dt).numpy()          # row-major b, odd k
            check_parity(oracle, got16, oracle.narrow(exact.astype(np.float32), is_bf16), is_bf16, what=f"{m}x{n}x{k} row-major b")
            wide = matmul(F, dev(F, a16, dt), dev(F, b16, dt), fl).numpy()            # kept as it was summed
            assert oracle.rel_l2(wide, exact) <= 1e-6


def test_batched_products(flint, oracle):
    """Batches on both operands, a right operand broadcast over a leading dimension, and a left
    operand that is a transposed view (what the composed attention of flint/operators.cc:148-230 multiplies)."""
    F = flint
    rng = np.random.default_rng(42)
    fl, h = F.DType.FLOAT, F.DType.FLOAT16
    a = randn(rng, (2, 3, 17, 40))
    b = randn(rng, (2, 3, 40, 24), 0.2)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert oracle.rel_l2(matmul(F, dev(F, a, fl), dev(F, b, fl), fl).numpy(), want) <= 1e-6
    b1 = randn(rng, (3, 40, 24), 0.2)                                         # one fewer leading dimension
    assert oracle.rel_l2(matmul(F, dev(F, a, fl), dev(F, b1, fl), fl).numpy(), a.astype(np.float64) @ b1.astype(np.float64)) <= 1e-6
    bb = randn(rng, (1, 3, 40, 24), 0.2)                                      # a leading 1 repeats
    assert oracle.rel_l2(matmul(F, dev(F, a, fl), dev(F, bb, fl), fl).numpy(), a.astype(np.float64) @ bb.astype(np.float64)) <= 1e-6
    # q k^T of an attention: k (heads, S, d) read as (heads, d, S); half operands, bias over columns
    q16 = oracle.narrow(randn(rng, (4, 33, 64)), False)
    k16 = oracle.narrow(randn(rng, (4, 50, 64)), False)
    kt = dev(F, k16, h).view_as((4, 64, 50), (50 * 64, 1, 64))
    got = matmul(F, dev(F, q16, h), kt, h).numpy()
    exact = oracle.widen(q16, False).astype(np.float64) @ oracle.widen(k16, False).astype(np.float64).transpose(0, 2, 1)
    check_parity(oracle, got, oracle.narrow(exact.astype(np.float32), False), False, what="batched q k^T")
    # a residual of out's shape on a batched product
    res = oracle.narrow(randn(rng, (4, 33, 50)), False)
    got = matmul(F, dev(F, q16, h), kt, h, dev(F, res, h)).numpy()
    check_parity(oracle, got, oracle.narrow((exact + oracle.widen(res, False)).astype(np.float32), False), False, what="batched + residual")


def test_what_is_not_a_product_is_refused(flint):
    F = flint
    a = F.Tensor.empty((4, 16), F.DType.FLOAT16)
    b = F.Tensor.empty((16, 8), F.DType.FLOAT16)
    out = F.Tensor.empty((4, 8), F.DType.FLOAT16)
    L = F.lib()
    f32 = F.Tensor.empty((4, 16), F.DType.FLOAT)
    assert L.fl_matmul(F.operators(), f32.raw(), b.raw(), out.raw()) == F.FL_ERROR_INVALID_ARG      # mixed operand types
    assert L.fl_matmul(F.operators(), a.raw(), F.Tensor.empty((15, 8), F.DType.FLOAT16).raw(), out.raw()) == F.FL_ERROR_INVALID_ARG
    assert b"disagree about k" in L.fl_get_last_error_message()
    assert L.fl_matmul(F.operators(), a.raw(), b.raw(), F.Tensor.empty((4, 9), F.DType.FLOAT16).raw()) == F.FL_ERROR_INVALID_ARG
    b3 = F.Tensor.empty((2, 16, 8), F.DType.FLOAT16)
    assert L.fl_matmul(F.operators(), a.raw(), b3.raw(), out.raw()) == F.FL_ERROR_INVALID_ARG       # b has more dimensions than a
    i8 = F.Tensor.empty((4, 16), F.DType.INT8)
    assert L.fl_matmul(F.operators(), i8.raw(), i8.raw(), out.raw()) == F.FL_ERROR_INVALID_ARG


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
