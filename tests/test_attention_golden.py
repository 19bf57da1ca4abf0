"""The CPU oracle's attention against outputs of the reference's own CPU fl_attention
(tests/golden/attention.npz, made by tests/golden/make_attention.py), and against the reference
library itself where it has been built."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention.npz")


@pytest.mark.parametrize("name", ["causal_gqa", "full_d128"])
def test_oracle_matches_the_reference_outputs(oracle, name):
    fx = np.load(GOLDEN)
    causal, is_bf16 = (bool(x) for x in fx[name + "_flags"])
    got = oracle.attention(fx[name + "_q"], fx[name + "_k"], fx[name + "_v"], causal, is_bf16)
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
