"""The block-step operators against tests/golden/block_steps.npz, outputs of the reference's own
CPU layer norm, RMS norm and swiglu (made by tests/golden/make_block_steps.py). The CPU tests hold
the oracle's restatements to the fixture; the GPU tests hold the kernels to it through the C ABI.
A float32 sum in another order (or the device's expf) can move a value across a 16-bit rounding
boundary now and then, hence "nearly all identical, the rest one step away"."""
import os

import numpy as np
import pytest

FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "block_steps.npz")


@pytest.fixture(scope="module")
def fx():
    return np.load(FIXTURE)


def close16(oracle, got, want, least=0.995):
    assert got.shape == want.shape
    assert np.mean(got == want) >= least, f"only {np.mean(got == want):.4f} identical"
    g, w = oracle.widen(got, True), oracle.widen(want, True)
    assert np.all(np.abs(g - w) <= np.maximum(np.abs(w), 2.0 ** -14) * 2.0 ** -7 * 1.01)


def test_oracle_layer_norm(oracle, fx):
    close16(oracle, oracle.layernorm_modulate(fx["ln_x"], None, None, float(fx["ln_eps"][0]), True), fx["ln_y"])


def test_oracle_rms_norm(oracle, fx):
    heads = int(fx["rms_heads"][0])
    head_dim = fx["rms_w"].shape[0]
    ones, zeros = np.ones((5, head_dim // 2), np.float32), np.zeros((5, head_dim // 2), np.float32)
    got = oracle.qk_norm_rope(fx["rms_qkv"], ones, zeros, heads, 1e-6, True, fx["rms_w"], fx["rms_w"])
    close16(oracle, got[:, :2 * heads * head_dim], fx["rms_y"], least=0.99)


def test_oracle_swiglu(oracle, fx):
    close16(oracle, oracle.swiglu(fx["swiglu_x"], True), fx["swiglu_y"])


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


@pytest.mark.gpu
def test_gpu_rms_norm(flint, oracle, fx):
    F = flint
    heads = int(fx["rms_heads"][0])
    head_dim = fx["rms_w"].shape[0]
    rows = fx["rms_qkv"].shape[0]
    ones, zeros = np.ones((rows // 2, head_dim // 2), np.float32), np.zeros((rows // 2, head_dim // 2), np.float32)
    t = dev(F, fx["rms_qkv"], F.DType.BFLOAT16)
    w = dev(F, fx["rms_w"], F.DType.BFLOAT16)
    F.qk_norm_rope(t, dev(F, ones, F.DType.FLOAT), dev(F, zeros, F.DType.FLOAT), heads, 1e-6, w, w)
    got = t.numpy()
    F.synchronize()
    close16(oracle, got[:, :2 * heads * head_dim], fx["rms_y"], least=0.99)
    assert np.array_equal(got[:, 2 * heads * head_dim:], fx["rms_qkv"][:, 2 * heads * head_dim:])


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["ln", "swiglu"])
def test_gpu_quantised_rows(flint, oracle, fx, which):
    """The fused kernels return e4m3 rows of the operator's output: dequantised, they sit within
    one e4m3 step of the reference's 16-bit values, and the row scales are amax / 448 of them."""
    F = flint
    bf = F.DType.BFLOAT16
    if which == "ln":
        codes, rs = F.fp8_layernorm_quantize(dev(F, fx["ln_x"], bf), None, None, float(fx["ln_eps"][0]))
        want16 = fx["ln_y"]
    else:
        codes, rs = F.fp8_swiglu_quantize(dev(F, fx["swiglu_x"], bf))
        want16 = fx["swiglu_y"]
    c, s = codes.numpy(), rs.numpy()
    F.synchronize()
    want = oracle.widen(want16, True)
    amax = np.abs(want).max(axis=1)
    assert np.all(np.abs(s - amax / 448.0) <= amax / 448.0 * 2.0 ** -7 * 1.01)
    got = oracle.decode_e4m3(c) * s[:, None]
    assert np.all(np.abs(got - want) <= np.maximum(np.abs(want), s[:, None]) * 2.0 ** -3 + 1e-30)
    assert oracle.rel_l2(got, want) <= 4e-2  # e4m3 has three mantissa bits
