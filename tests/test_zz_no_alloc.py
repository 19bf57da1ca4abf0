"""fl_fp8_linear_static -- the entry point for hosts that must not allocate on the device (the
whole card is budgeted to resident weights, or an allocation's device-wide stall is not
affordable mid-pass) -- against fl_fp8_linear, through the C ABI.

From five rows on both run the same quantiser and the same GEMM, one over the library's growable
arena and one over the fixed array compiled into the library, so their outputs must be identical
bit for bit. Two calls in a row with different shapes check that the array, which keeps the
previous call's contents, is not read where this call did not write it. A call at the array's
full size checks the property the entry point exists for: the card's free memory does not move.
The file is named to be collected last."""
import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def case(O, rng, m, n, k):
    x = O.narrow(randn(rng, (m, k)), True)
    codes, scales = O.quantize_fp8_rows(randn(rng, (n, k), 0.02))
    bias = O.narrow(randn(rng, (n,), 0.01), True)
    res = O.narrow(randn(rng, (m, n)), True)
    return x, codes, scales, bias, res


def test_static_entry_point_matches_fp8_linear_twice_in_a_row(flint, oracle):
    F = flint
    rng = np.random.default_rng(2024)
    bf = F.DType.BFLOAT16
    # a larger call first, then a smaller one that leaves most of the first one's bytes in place
    for (m, n, k, act) in [(520, 328, 1024, F.ACT_GELU_TANH), (130, 264, 208, F.ACT_NONE)]:
        x, codes, scales, bias, res = case(oracle, rng, m, n, k)
        xd, cd, sd, bd, rd = dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT), dev(F, bias, bf), dev(F, res, bf)
        out_static = F.Tensor.empty((m, n), bf)
        out_plain = F.Tensor.empty((m, n), bf)
        F.fp8_linear_static(xd, cd, sd, bd, rd, act, out_static)
        F.fp8_linear(xd, cd, sd, bd, rd, act, out_plain)
        got, plain = out_static.numpy(), out_plain.numpy()
        F.synchronize()
        assert np.array_equal(got, plain), f"{m}x{n}x{k}: the two entry points differ"
        check_parity(oracle, got, oracle.fp8_linear(x, codes, scales, bias, res, act), True, what=f"static {m}x{n}x{k}")


def test_static_entry_point_refuses_what_does_not_fit(flint, oracle):
    F = flint
    bf = F.DType.BFLOAT16
    k = 16384
    m = 1040  # m * k = 17 039 360 > 16 Mi elements
    xd = F.Tensor.empty((m, k), bf)
    cd = F.Tensor.empty((8, k), F.DType.FP8E4M3)
    sd = dev(F, np.ones(8, np.float32), F.DType.FLOAT)
    out = F.Tensor.empty((m, 8), bf)
    with pytest.raises(F.FlintError) as e:
        F.fp8_linear_static(xd, cd, sd, None, None, F.ACT_NONE, out)
    assert e.value.code == F.FL_ERROR_INVALID_ARG and "exceeds the static scratch" in e.value.message
    rows = F.Tensor.empty((65552, 16), bf)
    with pytest.raises(F.FlintError) as e:
        F.fp8_linear_static(rows, F.Tensor.empty((8, 16), F.DType.FP8E4M3), sd, None, None, F.ACT_NONE,
                            F.Tensor.empty((65552, 8), bf))
    assert e.value.code == F.FL_ERROR_INVALID_ARG and "rows exceed" in e.value.message


def test_static_entry_point_with_a_few_rows_matches_the_oracle(flint, oracle):
    """For one to four rows against a narrow weight fl_fp8_linear takes its one-launch few-row
    kernel, whose summation order differs; the static entry point runs the quantiser and the tile
    kernel, so here it is held to the oracle instead."""
    F = flint
    rng = np.random.default_rng(2025)
    bf = F.DType.BFLOAT16
    m, n, k = 2, 264, 1024
    x, codes, scales, bias, res = case(oracle, rng, m, n, k)
    out = F.Tensor.empty((m, n), bf)
    F.fp8_linear_static(dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT), dev(F, bias, bf),
                        dev(F, res, bf), F.ACT_GELU_TANH, out)
    got = out.numpy()
    F.synchronize()
    check_parity(oracle, got, oracle.fp8_linear(x, codes, scales, bias, res, F.ACT_GELU_TANH), True, what="static 2 rows")


def test_static_entry_point_leaves_the_cards_free_memory_alone(flint, oracle):
    """A call that fills the whole static array (m * k = 16 Mi elements, more than any call this
    file made before) between two readings of cudaMemGetInfo: every operand and the output exist
    before the first reading, so any byte the entry point allocated would show."""
    import torch
    F = flint
    bf = F.DType.BFLOAT16
    m, n, k = 4096, 256, 4096
    rng = np.random.default_rng(2026)
    x = oracle.narrow(randn(rng, (m, k)), True)
    codes, scales = oracle.quantize_fp8_rows(randn(rng, (n, k), 0.02))
    xd, cd, sd = dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT)
    out = F.Tensor.empty((m, n), bf)
    small = F.Tensor.empty((8, n), bf)
    F.fp8_linear_static(xd.view_as((8, k), (k, 1)), cd, sd, None, None, F.ACT_NONE, small)  # first call: kernels loaded
    F.synchronize()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    F.fp8_linear_static(xd, cd, sd, None, None, F.ACT_NONE, out)
    F.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes across the call"
    got = out.numpy()
    rows = slice(0, 64)
    check_parity(oracle, got[rows], oracle.fp8_linear(x[rows], codes, scales, None, None, 0), True, what="static, full array")
