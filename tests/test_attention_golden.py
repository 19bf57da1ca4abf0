"""The CPU oracle's attention against outputs of the reference's own CPU fl_attention
(tests/golden/attention.npz, made by tests/golden/make_attention.py), and against the reference
library itself where it has been built."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention.npz")


NAMES = ["causal_gqa", "full_d128", "block_causal", "block_diagonal"]


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_the_reference_outputs(oracle, name):
    fx = np.load(GOLDEN)
    mask, is_bf16, block = (int(x) for x in fx[name + "_flags"])
    got = oracle.attention(fx[name + "_q"], fx[name + "_k"], fx[name + "_v"], mask, bool(is_bf16), block)
    want = fx[name + "_y"].astype(np.float64)
    # The reference computes in float32 (flint/operators.cc:148-230); the oracle in float64.
    assert np.abs(got - want).max() < 5e-6
    assert oracle.rel_l2(got, want) < 2e-6


def test_causal_mask_is_aligned_to_the_bottom_right(oracle):
    """Query i sees keys 0 .. i + S - L (flint/capi.h:118-126): with L = 1 every key, and the first
    of L = S queries only key 0, whose value it returns."""
    rng = np.random.default_rng(5)
    q = oracle.narrow(rng.standard_normal((1, 1, 1, 64)).astype(np.float32), True)
    k = oracle.narrow(rng.standard_normal((1, 1, 9, 64)).astype(np.float32), True)
    v = oracle.narrow(rng.standard_normal((1, 1, 9, 64)).astype(np.float32), True)
    assert np.array_equal(oracle.attention(q, k, v, True, True), oracle.attention(q, k, v, False, True))
    q9 = oracle.narrow(rng.standard_normal((1, 1, 9, 64)).astype(np.float32), True)
    first = oracle.attention(q9, k, v, True, True)[0, 0, 0]
    assert np.allclose(first, oracle.widen(v, True)[0, 0, 0].astype(np.float64))


def test_restatement_against_the_reference_operator(oracle):
    if not oracle.have_ref():
        pytest.skip("the reference's CPU build is not present")
    rng = np.random.default_rng(11)
    for causal, (n, h, hk, L, S, d) in [(False, (1, 6, 2, 33, 47, 64)), (True, (2, 2, 1, 40, 40, 128)), (True, (1, 3, 3, 5, 21, 64))]:
        q = oracle.narrow(rng.standard_normal((n, h, L, d)).astype(np.float32), False)
        k = oracle.narrow(rng.standard_normal((n, hk, S, d)).astype(np.float32), False)
        v = oracle.narrow(rng.standard_normal((n, hk, S, d)).astype(np.float32), False)
        want = oracle.ref().attention(oracle.widen(q, False), oracle.widen(k, False), oracle.widen(v, False), causal)
        got = oracle.attention(q, k, v, causal, False)
        assert np.abs(got - want).max() < 5e-6


def test_block_masks_are_the_reference_ranges(oracle):
    """flint/cuda/attention.cu:165-179: under a block mask query p sees up to the end of its own block
    of `block_size` keys, from key 0 (block causal) or from the block's first key (block diagonal)."""
    keep = oracle.attention_keep(2, 4, 6, 10)   # positions 4..9, blocks of 4
    assert keep[0].tolist() == [True] * 8 + [False] * 2      # position 4: blocks 0 and 1
    assert keep[5].tolist() == [True] * 10                  # position 9: the last, ragged block too
    keep = oracle.attention_keep(3, 4, 10, 10)
    assert keep[5].tolist() == [False] * 4 + [True] * 4 + [False] * 2
    assert keep[9].tolist() == [False] * 8 + [True] * 2
    assert oracle.attention_keep(0, 0, 3, 3) is None
    if oracle.have_ref():
        # The reference's CPU device makes no block mask itself; the rows of one block of positions all
        # see the same keys, so they go through its unmasked fl_attention over exactly those keys.
        import importlib.util
        spec = importlib.util.spec_from_file_location("make_attention", os.path.join(os.path.dirname(GOLDEN), "make_attention.py"))
        gen = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(gen)
        rng = np.random.default_rng(12)
        for mask, block, (L, S) in [(2, 5, (23, 31)), (3, 7, (30, 30)), (2, 64, (40, 40))]:
            q = oracle.narrow(rng.standard_normal((1, 2, L, 64)).astype(np.float32), True)
            k = oracle.narrow(rng.standard_normal((1, 1, S, 64)).astype(np.float32), True)
            v = oracle.narrow(rng.standard_normal((1, 1, S, 64)).astype(np.float32), True)
            want = gen.reference_attention(oracle.ref(), oracle.widen(q, True), oracle.widen(k, True), oracle.widen(v, True), mask, block)
            assert np.abs(oracle.attention(q, k, v, mask, True, block) - want).max() < 5e-6
