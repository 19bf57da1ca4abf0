"""The C port of the oracle against the committed golden vectors, which were produced with the
reference's own CPU fl_matmul (tests/golden/make_golden.py). Runs without a GPU or the reference."""
import os

import numpy as np
import pytest

from helpers import check_parity

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantized_linear.npz")


@pytest.fixture(scope="module")
def fx():
    return np.load(GOLDEN)


@pytest.mark.parametrize("name", ["matmul_a", "matmul_b", "matmul_c"])
def test_port_reproduces_reference_matmul(oracle, fx, name):
    addend = fx[name + "_addend"] if name + "_addend" in fx else None
    y = oracle.fp8_matmul(fx[name + "_a"], fx[name + "_codes"], fx[name + "_scale"], addend, is_bf16=False, engine="port")
    # Only the order of the fp32 sums differs between the two engines: at most one half ulp flips.
    check_parity(oracle, y, fx[name + "_y"], False, rel=2e-4, ulps=1.0, what=name)
    assert np.mean(y != fx[name + "_y"]) < 0.01


@pytest.mark.parametrize("name", ["linear_a", "linear_b"])
def test_port_reproduces_reference_fp8_linear(oracle, fx, name):
    xc, xs = oracle.quantize_fp8_act(fx[name + "_x"], True)
    assert np.array_equal(xc, fx[name + "_xcodes"]) and np.array_equal(xs, fx[name + "_xscales"])
    bias = fx[name + "_bias"] if name + "_bias" in fx else None
    res = fx[name + "_res"] if name + "_res" in fx else None
    y = oracle.fp8_linear(fx[name + "_x"], fx[name + "_codes"], fx[name + "_scales"], bias, res,
                          int(fx[name + "_act"][0]), is_bf16=True, engine="port")
    check_parity(oracle, y, fx[name + "_y"], True, rel=1e-3, ulps=1.0, what=name)


@pytest.mark.parametrize("name", ["nvfp4_a", "nvfp4_b"])
def test_port_reproduces_reference_nvfp4_linear(oracle, fx, name):
    codes, sf, g = oracle.quantize_nvfp4_weight(fx[name + "_w"])
    assert np.array_equal(codes, fx[name + "_codes"]) and np.array_equal(sf, fx[name + "_sf"]) and g[0] == fx[name + "_g"][0]
    y = oracle.nvfp4_linear(fx[name + "_x"], fx[name + "_codes"], fx[name + "_sf"], fx[name + "_g"],
                            fx[name + "_bias"], None, int(fx[name + "_act"][0]), is_bf16=True, engine="port")
    check_parity(oracle, y, fx[name + "_y"], True, rel=1e-3, ulps=1.0, what=name)
