"""The tile kernel's stream-K schedule on the card: shapes whose last round of tiles would be partly
filled, so that the K stages of the last one-and-a-bit rounds are dealt out over all SMs and some
tiles are computed in two parts and summed through the workspace. Each case runs with that
schedule and with FLINT_SM100_NO_STREAM_K=1 (every tile whole); both must agree with the oracle to
the path's tolerance, the two must agree with each other to the last bits except in the tiles that
were cut (a different association of the same fp32 sum), and the stream-K result must be the same
bits on every run (the sum is head + tail whichever part arrived last)."""
import os

import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


class whole_tiles:
    """FLINT_SM100_NO_STREAM_K=1 for the duration (the library reads it on every call)."""

    def __enter__(self):
        self.old = os.environ.get("FLINT_SM100_NO_STREAM_K")
        os.environ["FLINT_SM100_NO_STREAM_K"] = "1"

    def __exit__(self, *exc):
        if self.old is None:
            os.environ.pop("FLINT_SM100_NO_STREAM_K", None)
        else:
            os.environ["FLINT_SM100_NO_STREAM_K"] = self.old


def plan(F, kind, m, n, k):
    import ctypes
    import torch
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    out = (ctypes.c_int32 * 8)()
    F.check(F.lib().fl_sm100_gemm_plan(kind, m, n, k, sms, 1, out))
    return list(out)


def compare(oracle, runs, want, is_bf16, what):
    sk_a, sk_b, dp = runs
    assert np.array_equal(sk_a, sk_b), f"{what}: two runs of the stream-K schedule differ"
    check_parity(oracle, sk_a, want, is_bf16, what=what + " (stream-K)")
    check_parity(oracle, dp, want, is_bf16, what=what + " (whole tiles)")
    a, b = oracle.widen(sk_a, is_bf16).astype(np.float64), oracle.widen(dp, is_bf16).astype(np.float64)
    assert oracle.rel_l2(a, b) <= 1e-3, f"{what}: the two schedules are {oracle.rel_l2(a, b):.2e} apart"
    same = float(np.mean(sk_a == dp))
    assert same >= 0.5, f"{what}: only {same:.2f} of the outputs are the same bits under both schedules"
    return same


# (m, n, k, act): pair tiles 256 x 256 (81 tiles on 74 pairs), single-CTA 128-wide tiles (160 on 148),
# and a ragged case whose edge tiles are partly outside the matrix; K long enough (48 stages) that
# the schedule takes its stream-K form
# ... and few tiles with a long K, every tile cut in two halves (8 pair tiles on 16 of the pairs; a ragged one)
@pytest.mark.parametrize("m,n,k,act", [(2304, 2304, 6144, 1), (20480, 128, 6144, 0), (2250, 2056, 6160, 0),
                                       (1024, 384, 12288, 1), (700, 392, 10368, 0)])
def test_fp8_linear_under_both_schedules(flint, oracle, m, n, k, act):
    F = flint
    p = plan(F, 2, m, n, k)
    if p[6] == 0:
        pytest.skip(f"this card's SM count gives the shape no stream-K part (plan {p})")
    rng = np.random.default_rng(m + n + k)
    x = oracle.narrow(randn(rng, (m, k)), True)
    codes, scales = oracle.quantize_fp8_rows(randn(rng, (n, k), 0.02))
    bias = oracle.narrow(randn(rng, (n,), 0.01), True)
    res = oracle.narrow(randn(rng, (m, n)), True)
    bf = F.DType.BFLOAT16
    ops = (dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT), dev(F, bias, bf), dev(F, res, bf))
    runs = [F.fp8_linear(*ops, act).numpy() for _ in range(2)]
    with whole_tiles():
        runs.append(F.fp8_linear(*ops, act).numpy())
    F.synchronize()
    same = compare(oracle, runs, oracle.fp8_linear(x, codes, scales, bias, res, act), True, f"fp8 {m}x{n}x{k}")
    print(f"fp8 {m}x{n}x{k}: plan {p}, {same:.3f} of the outputs identical under both schedules")


def test_nvfp4_linear_under_both_schedules(flint, oracle):
    F = flint
    m, n, k = 2304, 1728, 12288  # 9 x 9 pair tiles of 256 x 192, 48 K stages
    p = plan(F, 3, m, n, k)
    if p[6] == 0:
        pytest.skip(f"this card's SM count gives the shape no stream-K part (plan {p})")
    rng = np.random.default_rng(77)
    x = oracle.narrow(randn(rng, (m, k)), True)
    codes, sf, g = oracle.quantize_nvfp4_weight(randn(rng, (n, k), 0.02))
    bf = F.DType.BFLOAT16
    ops = (dev(F, x, bf), dev(F, codes, F.DType.FP4E2M1X2), dev(F, sf, F.DType.FP8E4M3), dev(F, g, F.DType.FLOAT))
    runs = [F.nvfp4_linear(*ops).numpy() for _ in range(2)]
    with whole_tiles():
        runs.append(F.nvfp4_linear(*ops).numpy())
    F.synchronize()
    compare(oracle, runs, oracle.nvfp4_linear(x, codes, sf, g), True, f"nvfp4 {m}x{n}x{k}")


@pytest.mark.parametrize("is_bf16", [True, False])
def test_16_bit_matmul_under_both_schedules(flint, oracle, is_bf16):
    F = flint
    m, n, k = 2304, 2304, 3072
    p = plan(F, 1 if is_bf16 else 0, m, n, k)
    if p[6] == 0:
        pytest.skip(f"this card's SM count gives the shape no stream-K part (plan {p})")
    rng = np.random.default_rng(78)
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    a = oracle.narrow(randn(rng, (m, k)), is_bf16)
    w = oracle.narrow(randn(rng, (n, k), 0.05), is_bf16)
    bias = oracle.narrow(randn(rng, (n,), 0.1), is_bf16)
    ops = (dev(F, a, dt), dev(F, w, dt), dev(F, bias, dt))
    runs = [F.linear_16(*ops).numpy() for _ in range(2)]
    with whole_tiles():
        runs.append(F.linear_16(*ops).numpy())
    F.synchronize()
    acc = oracle.gemm_f32_nt(oracle.widen(a, is_bf16), oracle.widen(w, is_bf16))
    compare(oracle, runs, oracle.epilogue(acc, bias=bias, out_is_bf16=is_bf16), is_bf16, f"16-bit {m}x{n}x{k}")


def test_counters_are_left_zero_between_launches(flint, oracle):
    """Back-to-back launches of different shapes share the workspace: the counters a launch counted
    up are zero again when it ends, so a following launch with other tiles sees a clean slate."""
    F = flint
    rng = np.random.default_rng(79)
    bf = F.DType.BFLOAT16
    outs, wants = [], []
    for (m, n, k) in [(2304, 2304, 6144), (2560, 2304, 6400), (2304, 2304, 6144), (20480, 128, 6144)]:
        x = oracle.narrow(randn(rng, (m, k)), True)
        codes, scales = oracle.quantize_fp8_rows(randn(rng, (n, k), 0.02))
        outs.append(F.fp8_linear(dev(F, x, bf), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT)))
        wants.append(oracle.fp8_linear(x, codes, scales, None, None, 0))
    for out, want in zip(outs, wants):
        check_parity(oracle, out.numpy(), want, True, what="back to back")
    F.synchronize()
