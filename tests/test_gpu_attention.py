"""GPU parity of fl_attention (masks none and causal) against the CPU oracle, through the C ABI.

The kernel rounds its probabilities to the operands' 16-bit type before the second product, as the
reference's kernels do (flint/cuda/attention.cu:30-70), and narrows its output once; the oracle
rounds nothing. Tolerance, written here: relative L2 error <= 5e-3 and every element within two
16-bit steps at the largest output magnitude."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention.npz")


def dtype_of(F, is_bf16):
    return F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16


def make(oracle, rng, n, h, hk, L, S, d, is_bf16, spread=1.0):
    q = oracle.narrow((rng.standard_normal((n, h, L, d)) * spread).astype(np.float32), is_bf16)
    k = oracle.narrow((rng.standard_normal((n, hk, S, d)) * spread).astype(np.float32), is_bf16)
    v = oracle.narrow(rng.standard_normal((n, hk, S, d)).astype(np.float32), is_bf16)
    return q, k, v


def run(F, q, k, v, causal, is_bf16, block_size=0):
    dt = dtype_of(F, is_bf16)
    tq, tk, tv = (F.Tensor.from_numpy(t, dt, F.Device.CUDA) for t in (q, k, v))
    out = F.attention(tq, tk, tv, int(causal), block_size)
    got = out.numpy()
    F.synchronize()
    return got


def check(oracle, got16, want, is_bf16, what):
    got = oracle.widen(got16, is_bf16).astype(np.float64)
    assert np.isfinite(got).all(), what
    err = oracle.rel_l2(got, want)
    step = oracle.ulp16_at(float(np.abs(want).max()), is_bf16)
    worst = float(np.abs(got - want).max())
    assert err <= 5e-3, f"{what}: rel L2 {err:.3e}"
    assert worst <= 2 * step, f"{what}: max abs {worst:.3e} > 2 steps of {step:.3e}"


SHAPES = [
    # n, heads, kv_heads, L, S, d
    (1, 1, 1, 128, 128, 128),
    (1, 2, 2, 128, 256, 64),
    (2, 3, 3, 200, 200, 128),
    (1, 4, 2, 77, 333, 64),      # grouped-query, ragged lengths
    (1, 8, 1, 1, 517, 128),      # one query (a decode step), multi-query
    (2, 2, 2, 300, 8, 64),       # fewer keys than a block
    (1, 2, 2, 513, 640, 128),
    (1, 2, 1, 640, 4224, 64),    # many blocks: the rings and the score buffers wrap many times
]


@pytest.mark.parametrize("n,h,hk,L,S,d", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("is_bf16", [True, False])
def test_parity(flint, oracle, n, h, hk, L, S, d, causal, is_bf16):
    if causal and S < L:
        pytest.skip("keys too few for the causal mask")
    rng = np.random.default_rng(900 + L + S + d + h)
    q, k, v = make(oracle, rng, n, h, hk, L, S, d, is_bf16)
    got = run(flint, q, k, v, causal, is_bf16)
    check(oracle, got, oracle.attention(q, k, v, causal, is_bf16), is_bf16, f"{(n, h, hk, L, S, d)} causal={causal}")


def test_peaked_scores(flint, oracle):
    """Scores far apart (|s| up to ~60 after scaling): the running maximum moves from block to block
    and most probabilities underflow to zero."""
    rng = np.random.default_rng(3)
    q, k, v = make(oracle, rng, 1, 2, 2, 256, 512, 128, True, spread=4.0)
    got = run(flint, q, k, v, False, True)
    check(oracle, got, oracle.attention(q, k, v, False, True), True, "peaked")


def test_transposed_operands(flint, oracle):
    """What a model hands in: (batch, length, heads, head_dim) tensors viewed as (batch, heads,
    length, head_dim) (flint/cuda/attention_test.cc:70-76), q, k and v being thirds of one fused
    projection, and out viewed the same way."""
    F = flint
    rng = np.random.default_rng(17)
    n, h, L, d = 2, 3, 150, 128
    qkv = oracle.narrow(rng.standard_normal((n, L, 3, h, d)).astype(np.float32), True)
    t = F.Tensor.from_numpy(qkv, F.DType.BFLOAT16, F.Device.CUDA)
    stride = (L * 3 * h * d, d, 3 * h * d, 1)
    tq, tk, tv = (t.view_as((n, h, L, d), stride, i * h * d) for i in range(3))
    out_store = F.Tensor.from_numpy(np.zeros((n, L, h, d), np.uint16), F.DType.BFLOAT16, F.Device.CUDA)
    out = out_store.view_as((n, h, L, d), (L * h * d, d, h * d, 1))
    F.attention(tq, tk, tv, F.MaskType.CAUSAL, 0, out)
    got = out_store.numpy().reshape(n, L, h, d).transpose(0, 2, 1, 3)
    F.synchronize()
    q, k, v = (np.ascontiguousarray(qkv[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))
    check(oracle, got, oracle.attention(q, k, v, True, True), True, "transposed")


@pytest.mark.parametrize("name", ["causal_gqa", "full_d128", "block_causal", "block_diagonal"])
def test_golden_vectors(flint, oracle, name):
    fx = np.load(GOLDEN)
    mask, is_bf16, block = (int(x) for x in fx[name + "_flags"])
    got = run(flint, fx[name + "_q"], fx[name + "_k"], fx[name + "_v"], mask, bool(is_bf16), block)
    check(oracle, got, fx[name + "_y"].astype(np.float64), is_bf16, name)


def test_what_is_not_a_mask_is_refused(flint, oracle):
    F = flint
    rng = np.random.default_rng(1)
    q, k, v = make(oracle, rng, 1, 2, 2, 16, 16, 64, True)
    tq, tk, tv = (F.Tensor.from_numpy(t, F.DType.BFLOAT16, F.Device.CUDA) for t in (q, k, v))
    for mask, block in [(F.MaskType.NONE, 4), (F.MaskType.CAUSAL, 4), (F.MaskType.BLOCK_CAUSAL, 0),
                        (F.MaskType.BLOCK_DIAGONAL, -1), (7, 0)]:
        with pytest.raises(F.FlintError):
            F.attention(tq, tk, tv, mask, block)
    # Keys too few for the causal masks, or not as many as queries for the diagonal one; a head_dim without a kernel.
    short = F.Tensor.from_numpy(k[:, :, :8].copy(), F.DType.BFLOAT16, F.Device.CUDA)
    for mask, block in [(F.MaskType.CAUSAL, 0), (F.MaskType.BLOCK_CAUSAL, 4), (F.MaskType.BLOCK_DIAGONAL, 4)]:
        with pytest.raises(F.FlintError):
            F.attention(tq, short, short, mask, block)
    q96, k96, v96 = make(oracle, rng, 1, 1, 1, 8, 8, 96, True)
    t96 = [F.Tensor.from_numpy(t, F.DType.BFLOAT16, F.Device.CUDA) for t in (q96, k96, v96)]
    with pytest.raises(F.FlintError):
        F.attention(*t96, F.MaskType.NONE, 0)


def test_step_size_properties(flint, oracle):
    """The denoise step's attention (2 x 24 heads x 4352 tokens x 128): rows of equal values come
    back as that value (the probabilities sum to one), doubling v doubles the output bit for bit,
    and one head agrees with the oracle."""
    rng = np.random.default_rng(23)
    n, h, L, d = 2, 24, 4352, 128
    q, k, v = make(oracle, rng, n, h, h, L, L, d, True)
    v[:, 0] = oracle.narrow(np.full((1,), 0.75, np.float32), True)[0]
    got = run(flint, q, k, v, False, True)
    const = oracle.widen(got[:, 0], True)
    assert np.abs(const - 0.75).max() <= oracle.ulp16_at(0.75, True)
    v2 = oracle.narrow(2.0 * oracle.widen(v, True), True)
    got2 = run(flint, q, k, v2, False, True)
    assert np.array_equal(oracle.widen(got2, True), 2.0 * oracle.widen(got, True))
    want = oracle.attention(q[1:, 5:6], k[1:, 5:6], v[1:, 5:6], False, True)
    check(oracle, got[1:, 5:6], want, True, "one head of the step")


def test_broadcast_views_are_refused_or_read_correctly(flint, oracle):
    """A stride of 0 over an extent above 1 (one k shared by both batch rows through an expanded
    view): q, k and out go through tensor maps, which cannot repeat a dimension, so such a view is
    refused with the reason; v, which is gathered with its true strides, may repeat, and a
    dimension of extent 1 may carry any stride."""
    F = flint
    rng = np.random.default_rng(31)
    n, h, L, S, d = 2, 2, 40, 72, 64
    q, k, v = make(oracle, rng, n, h, h, L, S, d, True)
    bf = F.DType.BFLOAT16
    tq = F.Tensor.from_numpy(q, bf, F.Device.CUDA)
    tk = F.Tensor.from_numpy(k, bf, F.Device.CUDA)
    k1 = F.Tensor.from_numpy(k[:1].copy(), bf, F.Device.CUDA)
    v1 = F.Tensor.from_numpy(v[:1].copy(), bf, F.Device.CUDA)
    k_shared = k1.view_as((n, h, S, d), (0, S * d, d, 1))
    v_shared = v1.view_as((n, h, S, d), (0, S * d, d, 1))
    with pytest.raises(F.FlintError) as e:
        F.attention(tq, k_shared, v_shared, F.MaskType.NONE, 0)
    assert e.value.code == F.FL_ERROR_INVALID_ARG and "stride of 0" in e.value.message
    out_shared = F.Tensor.empty((1, h, L, d), bf).view_as((n, h, L, d), (0, L * d, d, 1))
    tv = F.Tensor.from_numpy(v, bf, F.Device.CUDA)
    with pytest.raises(F.FlintError):
        F.attention(tq, tk, tv, F.MaskType.NONE, 0, out_shared)
    # v alone shared between the batch rows: read with its true strides
    got = F.attention(tq, tk, v_shared, F.MaskType.NONE, 0).numpy()
    F.synchronize()
    v_rep = np.concatenate([v[:1], v[:1]], axis=0)
    check(oracle, got, oracle.attention(q, k, v_rep, False, True), True, "v shared by the batch rows")
    # extent 1 with stride 0 indexes nothing
    q1 = F.Tensor.from_numpy(q[:1].copy(), bf, F.Device.CUDA).view_as((1, h, L, d), (0, L * d, d, 1))
    got1 = F.attention(q1, k1, v1, F.MaskType.NONE, 0).numpy()
    F.synchronize()
    check(oracle, got1, oracle.attention(q[:1], k[:1], v[:1], False, True), True, "batch of one, stride 0")


BLOCK_CASES = [
    # mask, block_size, n, heads, kv_heads, L, S, d
    (2, 64, 1, 2, 2, 300, 300, 64),     # block causal, blocks half a tile
    (2, 200, 1, 4, 2, 513, 700, 128),   # blocks that straddle tiles, more keys than queries, grouped heads
    (2, 1, 1, 1, 1, 130, 130, 64),      # blocks of one key: the causal mask
    (3, 128, 2, 2, 2, 512, 512, 128),   # block diagonal, blocks equal to tiles: every other block of keys is skipped
    (3, 48, 1, 3, 1, 333, 333, 64),     # ragged blocks inside tiles
    (3, 1000, 1, 2, 2, 260, 260, 128),  # one block covers everything: no mask
]


@pytest.mark.parametrize("mask,block,n,h,hk,L,S,d", BLOCK_CASES)
@pytest.mark.parametrize("is_bf16", [True, False])
def test_block_masks(flint, oracle, mask, block, n, h, hk, L, S, d, is_bf16):
    rng = np.random.default_rng(300 + mask * 10 + block)
    q, k, v = make(oracle, rng, n, h, hk, L, S, d, is_bf16)
    got = run(flint, q, k, v, mask, is_bf16, block)
    check(oracle, got, oracle.attention(q, k, v, mask, is_bf16, block), is_bf16, f"mask {mask} block {block}")
    if block == 1 and mask == 2:
        assert np.array_equal(got, run(flint, q, k, v, 1, is_bf16))      # the causal mask, bit for bit
    if block >= S and mask == 3:
        assert np.array_equal(got, run(flint, q, k, v, 0, is_bf16))      # no mask, bit for bit
