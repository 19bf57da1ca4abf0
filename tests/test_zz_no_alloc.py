"""fl_fp8_linear_static -- the entry point for hosts that must not allocate on the device (the
whole card is budgeted to resident weights, or an allocation's device-wide stall is not
affordable mid-pass) -- against fl_fp8_linear, through the C ABI.

Both run the same quantiser and the same GEMM, one over the library's growable arena and one over
the fixed array compiled into the library, so their outputs must be identical bit for bit. Two
calls in a row with different shapes check that the array, which keeps the previous call's
contents, is not read where this call did not write it. The file is named to be collected last."""
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
