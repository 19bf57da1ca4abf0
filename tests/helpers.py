"""Shared helpers of the parity tests: seeded inputs in the reference's style and the two
error measures the path is held to."""
import numpy as np


def randn(rng, shape, std=1.0):
    return (rng.standard_normal(shape) * std).astype(np.float32)


def random_codes(rng, n, k):
    """Codes from all of E4M3 but its two NaNs (flint/cuda/gemm_fp8_cutlass_test.cc:123-131)."""
    c = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    c[(c & 0x7F) == 0x7F] = 0x3C
    return c


def check_parity(O, got16, want16, is_bf16, rel=5e-3, ulps=2.0, what=""):
    """relative L2 <= rel and max abs error <= `ulps` output-type ulps at the output's scale."""
    got = O.widen(got16, is_bf16).astype(np.float64)
    want = O.widen(want16, is_bf16).astype(np.float64)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    r = O.rel_l2(got, want)
    scale = float(np.max(np.abs(want))) if want.size else 0.0
    ulp = O.ulp16_at(scale, is_bf16)
    max_abs = float(np.max(np.abs(got - want))) if want.size else 0.0
    assert r <= rel, f"{what}: relative L2 {r:.3e} > {rel}"
    assert max_abs <= ulps * ulp + 1e-30, f"{what}: max abs {max_abs:.4e} > {ulps} ulp ({ulp:.4e}) at scale {scale:.4e}"
    return r, max_abs / ulp if ulp else 0.0
