"""GPU parity of fl_fp8_swiglu_quantize (flint's swiglu fused with the per-row e4m3 quantiser of
the projection that follows it) against the CPU oracle, through the C ABI. The device's expf is not
correctly rounded, so a gated value can round to the neighbouring 16-bit value now and then: codes
are compared as dequantised values within one e4m3 step, nearly all of them identical."""
import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


@pytest.mark.parametrize("m,h", [(5, 8), (33, 1024), (7, 4104), (3, 12288), (2, 14344), (4, 20)])
@pytest.mark.parametrize("is_bf16", [True, False])
def test_codes_and_scales(flint, oracle, m, h, is_bf16):
    F = flint
    rng = np.random.default_rng(95 + m + h)
    x = oracle.narrow(randn(rng, (m, 2 * h)) * 3.0, is_bf16)
    x[0, :h] = oracle.narrow(np.full(h, -60.0, np.float32), is_bf16)  # a gate far below zero: silu -> -0
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    codes, row_scales = F.fp8_swiglu_quantize(dev(F, x, dt))
    c, s = codes.numpy(), row_scales.numpy()
    F.synchronize()
    y = oracle.swiglu(x, is_bf16)
    want_c, want_s = oracle.quantize_fp8_act(y, is_bf16)
    assert c.shape == (m, h) and s.shape == (m,)
    step = 2.0 ** -7 if is_bf16 else 2.0 ** -10
    assert np.all(np.abs(s - want_s) <= np.abs(want_s) * step * 1.01 + 1e-30)
    got = oracle.decode_e4m3(c) * s[:, None]
    want = oracle.decode_e4m3(want_c) * want_s[:, None]
    assert np.all(np.abs(got - want) <= np.maximum(np.abs(want), want_s[:, None]) * 2.0 ** -3 + 1e-30)
    assert np.mean(c == want_c) >= 0.98
    assert oracle.rel_l2(got, want) <= 5e-3


def test_gated_mlp_tail(flint, oracle):
    """swiglu -> quantise -> down projection with a residual, as a gated MLP's second half."""
    F = flint
    rng = np.random.default_rng(96)
    m, h, n = 200, 512, 264
    x = oracle.narrow(randn(rng, (m, 2 * h)) * 2.0, True)
    wc, ws = oracle.quantize_fp8_rows(randn(rng, (n, h), 0.02))
    res = oracle.narrow(randn(rng, (m, n)), True)
    bf = F.DType.BFLOAT16
    codes, row_scales = F.fp8_swiglu_quantize(dev(F, x, bf))
    out = F.Tensor.empty((m, n), bf)
    F.fp8_linear_quantized(codes, row_scales, dev(F, wc, F.DType.FP8E4M3), dev(F, ws, F.DType.FLOAT), None, dev(F, res, bf), 0, out)
    got = out.numpy()
    F.synchronize()
    want = oracle.fp8_linear(oracle.swiglu(x, True), wc, ws, None, res, 0, True)
    check_parity(oracle, got, want, True, what="swiglu_quantize -> linear_quantized")


def test_refusals(flint):
    F = flint
    bf = F.DType.BFLOAT16
    x = dev(F, np.zeros((4, 32), np.uint16), bf)
    with pytest.raises(F.FlintError):  # codes of the full width
        F.fp8_swiglu_quantize(x, F.Tensor.empty((4, 32), F.DType.FP8E4M3), F.Tensor.empty((4,), F.DType.FLOAT))
    with pytest.raises(F.FlintError):  # an odd last dimension
        F.fp8_swiglu_quantize(dev(F, np.zeros((4, 31), np.uint16), bf), F.Tensor.empty((4, 15), F.DType.FP8E4M3),
                              F.Tensor.empty((4,), F.DType.FLOAT))
    with pytest.raises(F.FlintError):  # row scales of the wrong length
        F.fp8_swiglu_quantize(x, F.Tensor.empty((4, 16), F.DType.FP8E4M3), F.Tensor.empty((3,), F.DType.FLOAT))
