"""GPU parity of fl_qk_norm_rope (per-head RMS norm of q and k and the rotation of their pairs, in
place on the fused projection's output) against the CPU oracle, through the C ABI. The mean of
squares is a float32 sum in another order than the oracle's, so a normalised value can round to the
neighbouring 16-bit value now and then: at most two 16-bit steps of a pair's length per element,
nearly all identical, and v untouched bit for bit."""
import numpy as np
import pytest

from helpers import randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def tables(rng, tokens, pairs):
    ang = rng.uniform(0, 2 * np.pi, (tokens, pairs)).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


@pytest.mark.parametrize("batch,tokens,heads,head_dim", [(2, 37, 3, 128), (1, 5, 2, 64), (3, 16, 1, 256), (2, 272, 24, 128)])
@pytest.mark.parametrize("is_bf16", [True, False])
@pytest.mark.parametrize("weights", [False, True])
def test_parity(flint, oracle, batch, tokens, heads, head_dim, is_bf16, weights):
    F = flint
    rng = np.random.default_rng(71 + tokens + heads + head_dim)
    rows, width = batch * tokens, 3 * heads * head_dim
    qkv = oracle.narrow(randn(rng, (rows, width)) * 2.0, is_bf16)
    qkv[1, :head_dim] = 0  # a zero head: rms = sqrt(eps), the result stays 0
    cos, sin = tables(rng, tokens, head_dim // 2)
    qw = oracle.narrow(1.0 + randn(rng, (head_dim,), 0.1), is_bf16) if weights else None
    kw = oracle.narrow(1.0 + randn(rng, (head_dim,), 0.1), is_bf16) if weights else None
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    t = dev(F, qkv.reshape(batch, tokens, width), dt)
    F.qk_norm_rope(t, dev(F, cos, F.DType.FLOAT), dev(F, sin, F.DType.FLOAT), heads, 1e-6,
                   dev(F, qw, dt) if weights else None, dev(F, kw, dt) if weights else None)
    got = t.numpy().reshape(rows, width)
    F.synchronize()
    want = oracle.qk_norm_rope(qkv, cos, sin, heads, 1e-6, is_bf16, qw, kw)
    assert np.array_equal(got[:, 2 * heads * head_dim:], qkv[:, 2 * heads * head_dim:])  # v
    g, w = oracle.widen(got, is_bf16), oracle.widen(want, is_bf16)
    assert np.all(np.isfinite(g))
    # A rotation keeps a pair's length, so that length (not the possibly cancelled result) is the
    # scale a one-step difference of a normalised input shows up at.
    step = 2.0 ** -7 if is_bf16 else 2.0 ** -10
    qk = slice(0, 2 * heads * head_dim)
    pair_len = np.repeat(np.sqrt((w[:, qk].reshape(rows, -1, 2) ** 2).sum(axis=2)), 2, axis=1)
    assert np.all(np.abs(g[:, qk] - w[:, qk]) <= np.maximum(pair_len, 2.0 ** -14) * step * 2.01)
    assert np.mean(got == want) >= 0.995
    assert oracle.rel_l2(g, w) <= 1e-3


def test_refusals(flint):
    F = flint
    bf = F.DType.BFLOAT16
    cos = dev(F, np.zeros((4, 64), np.float32), F.DType.FLOAT)
    with pytest.raises(F.FlintError):  # last dimension not 3 * heads * head_dim
        F.qk_norm_rope(dev(F, np.zeros((8, 3 * 2 * 128 + 8), np.uint16), bf), cos, cos, 2)
    with pytest.raises(F.FlintError):  # head_dim the kernel has no form for
        F.qk_norm_rope(dev(F, np.zeros((8, 3 * 2 * 96), np.uint16), bf), dev(F, np.zeros((4, 48), np.float32), F.DType.FLOAT),
                       dev(F, np.zeros((4, 48), np.float32), F.DType.FLOAT), 2)
    with pytest.raises(F.FlintError):  # rows that are not whole sequences
        F.qk_norm_rope(dev(F, np.zeros((6, 3 * 2 * 128), np.uint16), bf), cos, cos, 2)
    with pytest.raises(F.FlintError):  # tables of another width
        F.qk_norm_rope(dev(F, np.zeros((8, 3 * 2 * 128), np.uint16), bf), dev(F, np.zeros((4, 32), np.float32), F.DType.FLOAT),
                       dev(F, np.zeros((4, 32), np.float32), F.DType.FLOAT), 2)
