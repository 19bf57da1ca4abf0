"""GPU parity of the fused layer norm -> adaLN modulation -> per-row e4m3 quantiser
(fl_fp8_layernorm_quantize) and of fl_fp8_linear_quantized, through the C ABI, against the CPU
oracle's restatement of the reference's layerNorm and modulate.

The statistics are float32 sums whose order differs between the kernel and the oracle, so a
modulated value can land on the other side of a 16-bit rounding boundary now and then: the codes
are compared as dequantised values (within one 16-bit step of the row's scale, almost all of them
identical), the row scales within 2^-7 relative (one bfloat16 step), and the product built on them
with the tolerance of the path."""
import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def run_quantiser(F, x, scale, shift, eps, is_bf16):
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    codes, row_scales = F.fp8_layernorm_quantize(dev(F, x, dt), dev(F, scale, dt) if scale is not None else None,
                                                 dev(F, shift, dt) if shift is not None else None, eps)
    c, s = codes.numpy(), row_scales.numpy()
    F.synchronize()
    return c, s


def make(O, rng, m, k, groups, is_bf16, with_scale=True, with_shift=True):
    x = O.narrow(randn(rng, (m, k)) * 1.7 + 0.3, is_bf16)
    scale = O.narrow(randn(rng, (groups, k), 0.3), is_bf16) if with_scale else None
    shift = O.narrow(randn(rng, (groups, k), 0.2), is_bf16) if with_shift else None
    return x, scale, shift


@pytest.mark.parametrize("m,k,groups", [(8, 64, 1), (34, 3072, 2), (6, 16, 3), (12, 5000, 4), (4, 16392, 1), (10, 1040, 5)])
@pytest.mark.parametrize("is_bf16", [True, False])
def test_codes_and_scales(flint, oracle, m, k, groups, is_bf16):
    rng = np.random.default_rng(61 + m + k)
    for with_scale, with_shift in [(True, True), (True, False), (False, False)]:
        x, scale, shift = make(oracle, rng, m, k, groups, is_bf16, with_scale, with_shift)
        if m > 2:
            x[1] = x[1, 0]  # a constant row: variance 0, the normalised row is 0
        eps = 1e-6
        codes, row_scales = run_quantiser(flint, x, scale, shift, eps, is_bf16)
        h = oracle.layernorm_modulate(x, scale, shift, eps, is_bf16)
        want_codes, want_scales = oracle.quantize_fp8_act(h, is_bf16)
        assert codes.shape == (m, k) and row_scales.shape == (m,)
        step = 2.0 ** -7 if is_bf16 else 2.0 ** -10
        assert np.all(np.abs(row_scales - want_scales) <= np.abs(want_scales) * step * 1.01 + 1e-30)
        got = oracle.decode_e4m3(codes) * row_scales[:, None]
        want = oracle.decode_e4m3(want_codes) * want_scales[:, None]
        # one e4m3 step at the top of the row's range is amax / 8 * (1/2) ... compare per row
        tol = np.maximum(np.abs(want), want_scales[:, None]) * (2.0 ** -3) + 1e-30
        assert np.all(np.abs(got - want) <= tol)
        same = np.mean(codes == want_codes)
        assert same >= 0.98, f"only {same:.4f} of the codes are identical"
        assert oracle.rel_l2(got, want) <= 5e-3


def test_fused_equals_the_two_step_path(flint, oracle):
    """With the modulation switched off the kernel's 16-bit row is the plain layer norm; the codes
    then equal quantising the oracle's layer norm except where a statistic's last bit moved a
    16-bit rounding, and the product through fl_fp8_linear_quantized meets the path's tolerance."""
    F = flint
    rng = np.random.default_rng(62)
    m, n, k = 300, 264, 1040
    x, scale, shift = make(oracle, rng, m, k, 2, True)
    w = randn(rng, (n, k), 0.02)
    wc, ws = oracle.quantize_fp8_rows(w)
    bias = oracle.narrow(randn(rng, (n,), 0.01), True)
    res = oracle.narrow(randn(rng, (m, n)), True)
    bf = F.DType.BFLOAT16
    codes, row_scales = F.fp8_layernorm_quantize(dev(F, x, bf), dev(F, scale, bf), dev(F, shift, bf), 1e-6)
    out = F.Tensor.empty((m, n), bf)
    F.fp8_linear_quantized(codes, row_scales, dev(F, wc, F.DType.FP8E4M3), dev(F, ws, F.DType.FLOAT), dev(F, bias, bf),
                           dev(F, res, bf), F.ACT_GELU_TANH, out)
    got = out.numpy()
    F.synchronize()
    h = oracle.layernorm_modulate(x, scale, shift, 1e-6, True)
    want = oracle.fp8_linear(h, wc, ws, bias, res, oracle.ACT_GELU_TANH, True)
    check_parity(oracle, got, want, True, what="layernorm_quantize -> linear_quantized")
    # and the quantised entry agrees bit for bit with fl_fp8_linear on the same 16-bit rows
    direct = F.fp8_linear(dev(F, h, bf), dev(F, wc, F.DType.FP8E4M3), dev(F, ws, F.DType.FLOAT), dev(F, bias, bf),
                          dev(F, res, bf), F.ACT_GELU_TANH).numpy()
    c2, s2 = F.quantize_fp8_activation(dev(F, h, bf))
    out2 = F.Tensor.empty((m, n), bf)
    F.fp8_linear_quantized(c2, s2, dev(F, wc, F.DType.FP8E4M3), dev(F, ws, F.DType.FLOAT), dev(F, bias, bf),
                           dev(F, res, bf), F.ACT_GELU_TANH, out2)
    assert np.array_equal(out2.numpy(), direct)


def test_refusals(flint):
    F = flint
    bf = F.DType.BFLOAT16
    x = dev(F, np.zeros((6, 32), np.uint16), bf)
    codes = F.Tensor.empty((6, 32), F.DType.FP8E4M3)
    rs = F.Tensor.empty((6,), F.DType.FLOAT)
    with pytest.raises(F.FlintError):  # groups that do not divide the rows
        F.fp8_layernorm_quantize(x, dev(F, np.zeros((4, 32), np.uint16), bf), None, 1e-6, codes, rs)
    with pytest.raises(F.FlintError):  # a scale of another width
        F.fp8_layernorm_quantize(x, dev(F, np.zeros((2, 16), np.uint16), bf), None, 1e-6, codes, rs)
    with pytest.raises(F.FlintError):  # scale and shift of different group counts
        F.fp8_layernorm_quantize(x, dev(F, np.zeros((2, 32), np.uint16), bf), dev(F, np.zeros((3, 32), np.uint16), bf), 1e-6, codes, rs)
    with pytest.raises(F.FlintError):  # row scales of the wrong length
        F.fp8_layernorm_quantize(x, None, None, 1e-6, codes, F.Tensor.empty((5,), F.DType.FLOAT))
    with pytest.raises(F.FlintError):  # negative eps
        F.fp8_layernorm_quantize(x, None, None, -1.0, codes, rs)


def test_modulation_vectors_as_column_slices(flint, oracle):
    """scale and shift are usually chunks of one projection's output (groups, 6 k): a (groups, k)
    view with the wide tensor's row stride gives the same codes as contiguous copies."""
    F = flint
    rng = np.random.default_rng(63)
    m, k, groups = 12, 1040, 3
    bf = F.DType.BFLOAT16
    x = oracle.narrow(randn(rng, (m, k)) * 1.3, True)
    wide = oracle.narrow(randn(rng, (groups, 6 * k), 0.3), True)
    scale, shift = wide[:, k:2 * k].copy(), wide[:, 3 * k:4 * k].copy()
    wide_dev = dev(F, wide, bf)
    scale_view = wide_dev.view_as((groups, k), (6 * k, 1), k)
    shift_view = wide_dev.view_as((groups, k), (6 * k, 1), 3 * k)
    c1, s1 = F.fp8_layernorm_quantize(dev(F, x, bf), scale_view, shift_view, 1e-6)
    c2, s2 = F.fp8_layernorm_quantize(dev(F, x, bf), dev(F, scale, bf), dev(F, shift, bf), 1e-6)
    assert np.array_equal(c1.numpy(), c2.numpy()) and np.array_equal(s1.numpy(), s2.numpy())
    F.synchronize()
