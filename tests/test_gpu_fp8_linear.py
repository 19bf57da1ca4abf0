"""GPU parity of fl_fp8_linear (dynamic per-token e4m3 activation x e4m3 weight, per-channel
scales, fused bias / GELU-tanh / residual) against the CPU oracle, through the C ABI.
Tolerance: relative L2 <= 5e-3 and max abs error <= 2 bf16 ulp at the output's scale."""
import os

import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def make_case(O, rng, m, n, k, is_bf16=True, bias=False, residual=False, per_tensor=False):
    x = O.narrow(randn(rng, (m, k)), is_bf16)
    w = randn(rng, (n, k), 0.02)
    if per_tensor:
        codes, scales = O.quantize_fp8_tensor(w)
    else:
        codes, scales = O.quantize_fp8_rows(w)
    b = O.narrow(randn(rng, (n,), 0.01), is_bf16) if bias else None
    r = O.narrow(randn(rng, (m, n)), is_bf16) if residual else None
    return x, codes, scales, b, r


def run(F, x, codes, scales, bias, res, act, is_bf16=True):
    dt = F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16
    out = F.fp8_linear(dev(F, x, dt), dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT),
                       dev(F, bias, dt) if bias is not None else None, dev(F, res, dt) if res is not None else None, act)
    y = out.numpy()
    F.synchronize()
    return y


def test_activation_quantiser_is_bit_exact(flint, oracle):
    rng = np.random.default_rng(21)
    F = flint
    for is_bf16 in (True, False):
        for (m, k) in [(5, 16), (130, 208), (257, 3072)]:
            x = oracle.narrow(randn(rng, (m, k)), is_bf16)
            x[min(3, m - 1)] = 0  # a zero row: scale 0, codes 0
            x[0, 0] = oracle.narrow(np.array([1e4], np.float32), is_bf16)[0]  # an outlier row
            codes, scales = F.quantize_fp8_activation(dev(F, x, F.DType.BFLOAT16 if is_bf16 else F.DType.FLOAT16))
            want_c, want_s = oracle.quantize_fp8_act(x, is_bf16)
            assert np.array_equal(scales.numpy().view(np.uint32), want_s.view(np.uint32))
            assert np.array_equal(codes.numpy(), want_c)


def test_weight_quantiser_is_bit_exact(flint, oracle):
    rng = np.random.default_rng(22)
    F = flint
    w = randn(rng, (72, 208), 0.02)
    w[7] = 0
    codes, scales = F.quantize_fp8_rows(dev(F, w, F.DType.FLOAT))
    want_c, want_s = oracle.quantize_fp8_rows(w)
    assert np.array_equal(scales.numpy().view(np.uint32), want_s.view(np.uint32))
    assert np.array_equal(codes.numpy(), want_c)


EDGE = [(1, 8, 16), (2, 16, 16), (17, 128, 64), (129, 264, 96), (64, 64, 80), (300, 200, 256), (513, 64, 64),
        (128, 256, 128), (1, 3072, 3072), (16, 12288, 3072), (256, 1032, 144)]


@pytest.mark.parametrize("m,n,k", EDGE)
def test_edge_shapes(flint, oracle, m, n, k):
    rng = np.random.default_rng(100 + m + n + k)
    x, codes, scales, b, r = make_case(oracle, rng, m, n, k, bias=True, residual=True)
    got = run(flint, x, codes, scales, b, r, 0)
    want = oracle.fp8_linear(x, codes, scales, b, r, 0)
    check_parity(oracle, got, want, True, what=f"{m}x{n}x{k}")


@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("is_bf16", [True, False])
def test_epilogue_variants(flint, oracle, act, is_bf16):
    rng = np.random.default_rng(31 + act)
    for bias, residual, per_tensor in [(False, False, False), (True, False, True), (False, True, False), (True, True, False)]:
        x, codes, scales, b, r = make_case(oracle, rng, 200, 320, 192, is_bf16, bias, residual, per_tensor)
        got = run(flint, x, codes, scales, b, r, act, is_bf16)
        want = oracle.fp8_linear(x, codes, scales, b, r, act, is_bf16)
        check_parity(oracle, got, want, is_bf16, what=f"act={act} bias={bias} res={residual} pt={per_tensor}")


@pytest.mark.parametrize("m,n,k", [(1, 18432, 3072), (2, 264, 80), (3, 4096, 12288), (4, 72, 3088), (2, 8, 16),
                                   (4, 1184, 592), (2, 136, 4112), (3, 72, 8208)])
@pytest.mark.parametrize("is_bf16", [True, False])
def test_few_rows(flint, oracle, m, n, k, is_bf16):
    """One to four rows take the one-launch kernel that quantises the rows itself: every epilogue
    form, k that is not a multiple of a step, a zero row, per-tensor scale."""
    rng = np.random.default_rng(51 + m + n + k)
    for act, bias, residual, per_tensor in [(0, False, False, False), (1, True, False, False), (0, True, True, True),
                                            (1, False, True, False)]:
        x, codes, scales, b, r = make_case(oracle, rng, m, n, k, is_bf16, bias, residual, per_tensor)
        if m > 1:
            x[m - 1] = 0
        got = run(flint, x, codes, scales, b, r, act, is_bf16)
        want = oracle.fp8_linear(x, codes, scales, b, r, act, is_bf16)
        check_parity(oracle, got, want, is_bf16, what=f"few rows {m}x{n}x{k} act={act} bias={bias} res={residual}")


@pytest.mark.parametrize("m,n,k", [(5, 3080, 2064), (32, 3072, 2048), (17, 4104, 4096), (4, 3072, 2304), (2, 8200, 2048),
                                   (16, 19080, 3072), (9, 3072, 12288)])
@pytest.mark.parametrize("is_bf16", [True, False])
def test_few_rows_on_the_tensor_cores(flint, oracle, m, n, k, is_bf16):
    """At most 32 rows against a wide, deep weight: the quantiser's codes go to the kernel that puts
    the weight on the instruction's M side. Every epilogue form, a ragged last block of channels, k
    that ends inside a 32-byte step and inside a stage, a zero row, more CTAs than SMs."""
    rng = np.random.default_rng(61 + m + n + k)
    for act, bias, residual, per_tensor in [(0, False, False, False), (1, True, False, False), (0, True, True, True),
                                            (1, False, True, False)]:
        x, codes, scales, b, r = make_case(oracle, rng, m, n, k, is_bf16, bias, residual, per_tensor)
        if m > 1:
            x[m - 1] = 0
        got = run(flint, x, codes, scales, b, r, act, is_bf16)
        want = oracle.fp8_linear(x, codes, scales, b, r, act, is_bf16)
        check_parity(oracle, got, want, is_bf16, what=f"few rows {m}x{n}x{k} act={act} bias={bias} res={residual}")


def test_few_rows_on_the_tensor_cores_match_the_tile_kernel(flint, oracle):
    """The same rows alone (the few-row kernel) and inside 64 rows (the tile kernel), with a weight
    of +-1 so that every partial sum is exact: the two epilogues agree to the last bit, through
    fl_fp8_linear, fl_fp8_linear_static and fl_fp8_linear_quantized."""
    rng = np.random.default_rng(62)
    F = flint
    n, k = 3080, 2064
    x = oracle.narrow(randn(rng, (64, k)), True)
    codes = np.where(rng.random((n, k)) < 0.5, 0x38, 0xb8).astype(np.uint8)
    scales = (0.25 + rng.random(n)).astype(np.float32)
    bias = oracle.narrow(randn(rng, (n,)), True)
    res = oracle.narrow(randn(rng, (64, n)), True)
    few = run(F, x[:8], codes, scales, bias, res[:8], 1)
    many = run(F, x, codes, scales, bias, res, 1)
    assert np.array_equal(few, many[:8])
    bf = F.DType.BFLOAT16
    cd, sd = dev(F, codes, F.DType.FP8E4M3), dev(F, scales, F.DType.FLOAT)
    out = F.Tensor.empty((8, n), bf)
    F.fp8_linear_static(dev(F, x[:8], bf), cd, sd, dev(F, bias, bf), dev(F, res[:8], bf), 1, out)
    assert np.array_equal(out.numpy(), few)
    a_codes, a_scales = oracle.quantize_fp8_act(x[:8], True)
    out2 = F.Tensor.empty((8, n), bf)
    F.fp8_linear_quantized(dev(F, a_codes, F.DType.FP8E4M3), dev(F, a_scales, F.DType.FLOAT), cd, sd, dev(F, bias, bf),
                           dev(F, res[:8], bf), 1, out2)
    assert np.array_equal(out2.numpy(), few)


@pytest.mark.parametrize("m,rows_per_group,n,k", [(768, 256, 264, 320), (1152, 512, 520, 3072), (8704, 4352, 3072, 512)])
def test_row_groups_equal_one_product_per_group(flint, oracle, m, rows_per_group, n, k):
    """fl_fp8_linear_quantized_grouped: rows in groups, each with its own per-channel scales and bias
    (a gate per image folded into them). Equal to the last bit to one product per group, and
    within the path's tolerance of the oracle; a group size that is no multiple of 256 is refused."""
    F = flint
    rng = np.random.default_rng(71 + m + n)
    groups = -(-m // rows_per_group)
    x = oracle.narrow(randn(rng, (m, k)), True)
    a_codes, a_scales = oracle.quantize_fp8_act(x, True)
    w = randn(rng, (n, k), 0.02)
    wc, ws = oracle.quantize_fp8_rows(w)
    gate = (0.5 + rng.random((groups, n))).astype(np.float32)
    scales = (gate * ws[None, :]).astype(np.float32)
    bias = oracle.narrow(randn(rng, (groups, n), 0.1), True)
    res = oracle.narrow(randn(rng, (m, n)), True)
    bf = F.DType.BFLOAT16
    cd, rsd, wd = dev(F, a_codes, F.DType.FP8E4M3), dev(F, a_scales, F.DType.FLOAT), dev(F, wc, F.DType.FP8E4M3)
    out = F.Tensor.empty((m, n), bf)
    F.fp8_linear_quantized_grouped(cd, rsd, wd, dev(F, scales, F.DType.FLOAT), dev(F, bias, bf), dev(F, res, bf), 1,
                                   rows_per_group, out)
    got = out.numpy()
    for g in range(groups):
        r0, r1 = g * rows_per_group, min(m, (g + 1) * rows_per_group)
        part = F.Tensor.empty((r1 - r0, n), bf)
        F.fp8_linear_quantized(dev(F, a_codes[r0:r1], F.DType.FP8E4M3), dev(F, a_scales[r0:r1], F.DType.FLOAT), wd,
                               dev(F, scales[g], F.DType.FLOAT), dev(F, bias[g], bf), dev(F, res[r0:r1], bf), 1, part)
        assert np.array_equal(part.numpy(), got[r0:r1]), f"group {g}"
        want = oracle.fp8_linear_quantized(a_codes[r0:r1], a_scales[r0:r1], wc, scales[g], bias[g], res[r0:r1],
                                           oracle.ACT_GELU_TANH)
        check_parity(oracle, got[r0:r1], want, True, what=f"group {g}")
    with pytest.raises(F.FlintError):
        F.fp8_linear_quantized_grouped(cd, rsd, wd, dev(F, scales, F.DType.FLOAT), dev(F, bias, bf), dev(F, res, bf), 1, 100, out)


def test_few_rows_match_the_tile_path_quantiser(flint, oracle):
    """The in-kernel quantiser of the few-row kernel is the activation quantiser's arithmetic: with
    a weight of exact small integers the two paths (m = 4 and the same rows inside m = 64) agree
    to the last bit."""
    rng = np.random.default_rng(52)
    F = flint
    n, k = 136, 1040
    x = oracle.narrow(randn(rng, (64, k)), True)
    codes = np.where(rng.random((n, k)) < 0.5, 0x38, 0xb8).astype(np.uint8)  # +-1
    scales = np.full(n, 0.5, np.float32)
    few = run(F, x[:4], codes, scales, None, None, 0)
    many = run(F, x, codes, scales, None, None, 0)
    assert np.array_equal(few, many[:4])


def test_zero_rows_and_outliers(flint, oracle):
    rng = np.random.default_rng(41)
    x, codes, scales, b, r = make_case(oracle, rng, 96, 136, 128, bias=True)
    x[5] = 0
    x[9, 17] = oracle.narrow(np.array([1e4], np.float32), True)[0]
    codes[3] = 0
    scales[3] = 0.0
    got = run(flint, x, codes, scales, b, None, 0)
    want = oracle.fp8_linear(x, codes, scales, b, None, 0)
    assert np.array_equal(got[5], want[5])  # zero activation row -> bias only
    check_parity(oracle, got, want, True, what="zeros/outliers")


def test_all_codes_sweep(flint, oracle):
    """Every finite e4m3 code on both sides with unit scales: products are exact in fp32."""
    F = flint
    finite = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    rng = np.random.default_rng(42)
    codes = rng.choice(finite, size=(256, 256))
    # An activation whose every row's amax is 448 quantises to its own codes with scale 1.
    table = oracle.e4m3_decode_table()
    xa = rng.choice(finite, size=(128, 256))
    xa[:, 0] = 0x7E
    vals = table[xa] / 64.0  # keep sums small enough for bf16-exact inputs; scale = 1/64
    x = oracle.narrow(vals.astype(np.float32), True)
    got = run(F, x, codes, np.ones(256, np.float32), None, None, 0)
    want = oracle.fp8_linear(x, codes, np.ones(256, np.float32))
    check_parity(oracle, got, want, True, what="all codes")


@pytest.mark.parametrize("name", ["linear_a", "linear_b"])
def test_golden_vectors(flint, oracle, name):
    fx = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantized_linear.npz"))
    bias = fx[name + "_bias"] if name + "_bias" in fx else None
    res = fx[name + "_res"] if name + "_res" in fx else None
    got = run(flint, fx[name + "_x"], fx[name + "_codes"], fx[name + "_scales"], bias, res, int(fx[name + "_act"][0]))
    check_parity(oracle, got, fx[name + "_y"], True, what=name)


def test_config1_single_fp8_linear(flint, oracle):
    """X bf16 [4096,3072] ~N(0,1), W ~N(0,0.02) e4m3 per-row scales, bias ~N(0,0.01), seed 0."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(4096, 3072, generator=g).bfloat16().view(torch.uint16).numpy()
    w = (0.02 * torch.randn(3072, 3072, generator=g)).numpy()
    b = (0.01 * torch.randn(3072, generator=g)).bfloat16().view(torch.uint16).numpy()
    codes, scales = oracle.quantize_fp8_rows(w)
    got = run(flint, x, codes, scales, b, None, 0)
    want = oracle.fp8_linear(x, codes, scales, b, None, 0)
    r, u = check_parity(oracle, got, want, True, what="config 1")
    print(f"config 1: rel L2 {r:.3e}, max {u:.2f} ulp")


def test_config2_mlp_each_linear_and_chained(flint, oracle):
    """Qwen-Image-shaped FP8 MLP: up 3072->12288 + GELU-tanh, down 12288->3072 + residual X.
    Each linear is checked on identical inputs; the chain (the second GEMM fed the GPU's own H
    against the oracle fed its own H) is checked to the same bound."""
    import torch
    F = flint
    g = torch.Generator(device="cpu").manual_seed(0)
    m = 4352
    x = torch.randn(m, 3072, generator=g).bfloat16().view(torch.uint16).numpy()
    w_up = (0.02 * torch.randn(12288, 3072, generator=g)).numpy()
    w_down = (0.02 * torch.randn(3072, 12288, generator=g)).numpy()
    up_c, up_s = oracle.quantize_fp8_rows(w_up)
    dn_c, dn_s = oracle.quantize_fp8_rows(w_down)
    bf = F.DType.BFLOAT16
    xd = dev(F, x, bf)
    h = F.fp8_linear(xd, dev(F, up_c, F.DType.FP8E4M3), dev(F, up_s, F.DType.FLOAT), None, None, F.ACT_GELU_TANH)
    y = F.fp8_linear(h, dev(F, dn_c, F.DType.FP8E4M3), dev(F, dn_s, F.DType.FLOAT), None, xd, F.ACT_NONE)
    h_gpu, y_gpu = h.numpy(), y.numpy()
    F.synchronize()
    h_ref = oracle.fp8_linear(x, up_c, up_s, None, None, oracle.ACT_GELU_TANH)
    check_parity(oracle, h_gpu, h_ref, True, what="up + GELU")
    y_same_in = oracle.fp8_linear(h_gpu, dn_c, dn_s, None, x, oracle.ACT_NONE)
    check_parity(oracle, y_gpu, y_same_in, True, what="down + residual (same H)")
    y_chain = oracle.fp8_linear(h_ref, dn_c, dn_s, None, x, oracle.ACT_NONE)
    check_parity(oracle, y_gpu, y_chain, True, what="chained MLP")


def test_linearity_in_the_weight_scale_at_full_size(flint, oracle):
    """A size-independent property at the benchmark's size: doubling every channel scale doubles
    the product exactly (power-of-two scaling commutes with every rounding involved)."""
    rng = np.random.default_rng(51)
    F = flint
    m, n, k = 4352, 3072, 3072
    x = oracle.narrow(randn(rng, (m, k)), True)
    codes = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3C
    scales = (rng.random(n).astype(np.float32) + 0.5) * np.float32(1e-3)
    xd, cd = dev(F, x, F.DType.BFLOAT16), dev(F, codes, F.DType.FP8E4M3)
    y1 = F.fp8_linear(xd, cd, dev(F, scales, F.DType.FLOAT)).numpy()
    y2 = F.fp8_linear(xd, cd, dev(F, scales * 2, F.DType.FLOAT)).numpy()
    assert np.array_equal(oracle.widen(y1, True) * 2, oracle.widen(y2, True))
    # and a row subsample against the oracle
    rows = rng.choice(m, size=64, replace=False)
    want = oracle.fp8_linear(x[rows], codes, scales)
    check_parity(oracle, y1[rows], want, True, what="row subsample")
