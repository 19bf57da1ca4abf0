"""GPU parity of the reference-compatible entry points fl_fp8_matmul / fl_fp8_matmul_add, through
the C ABI, restating the reference's own kernel tests (flint/cuda/gemm_fp8_cutlass_test.cc) with
the CPU oracle in the place of the reference's half GEMM."""
import os

import numpy as np
import pytest

from helpers import check_parity, random_codes

pytestmark = pytest.mark.gpu

K_SCALE = np.float32(0.0137)  # not a power of two (gemm_fp8_cutlass_test.cc:162)


def f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def from_f16(b):
    return np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def run(F, a16, codes, scale, addend=None, dtype=None, expand=True):
    dtype = dtype or F.DType.FLOAT16
    a = dev(F, a16, dtype)
    w = dev(F, codes, F.DType.FP8E4M3)
    s = dev(F, np.asarray(scale, np.float32).reshape(1), F.DType.FLOAT)
    if addend is None:
        out = F.fp8_matmul(a, w, s)
    else:
        out = F.fp8_matmul_add(a, w, s, dev(F, addend, dtype), expand=expand)
    y = out.numpy()
    F.synchronize()
    return y


SHAPES = [(128, 128, 64), (1, 128, 64), (1, 5120, 3072), (1, 8, 16), (2, 16, 16), (17, 128, 64), (128, 264, 64),
          (129, 264, 96), (64, 64, 80), (3, 8, 32), (300, 200, 256), (1, 8, 4096), (512, 64, 64), (513, 64, 64)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_shapes(flint, oracle, m, n, k):
    # gemm_fp8_cutlass_test.cc:182-211
    rng = np.random.default_rng(7 + m * 131 + n * 17 + k)
    a = f16(rng.standard_normal((m, k)))
    codes = random_codes(rng, n, k)
    got = run(flint, a, codes, K_SCALE)
    assert got.shape == (m, n)
    want = oracle.fp8_matmul(a, codes, [K_SCALE])
    check_parity(oracle, got, want, False, what=f"{m}x{n}x{k}")


def test_availability_on_the_card(flint):
    assert flint.fp8_available(flint.Device.CUDA)
    assert flint.nvfp4_available(flint.Device.CUDA)
    assert not flint.fp8_available(flint.Device.CPU)


def test_batch_axes_fold_bit_exactly(flint, oracle):
    # gemm_fp8_cutlass_test.cc:213-230
    rng = np.random.default_rng(11)
    codes = random_codes(rng, 64, 128)
    a3 = f16(rng.standard_normal((2, 3, 128)))
    out3 = run(flint, a3, codes, 0.5)
    assert out3.shape == (2, 3, 64)
    flat = run(flint, a3.reshape(-1, 128), codes, 0.5)
    assert np.array_equal(out3.reshape(-1, 64), flat)
    a4 = f16(rng.standard_normal((2, 3, 5, 128)))
    assert run(flint, a4, codes, 0.5).shape == (2, 3, 5, 64)


def test_reused_weight(flint, oracle):
    # gemm_fp8_cutlass_test.cc:232-246
    rng = np.random.default_rng(12)
    F = flint
    codes = random_codes(rng, 128, 256)
    w = dev(F, codes, F.DType.FP8E4M3)
    s = dev(F, np.array([K_SCALE], np.float32), F.DType.FLOAT)
    for m in (1, 7, 64):
        a = f16(rng.standard_normal((m, 256)))
        got = F.fp8_matmul(dev(F, a, F.DType.FLOAT16), w, s).numpy()
        check_parity(oracle, got, oracle.fp8_matmul(a, codes, [K_SCALE]), False, what=f"m={m}")


def test_scale_applied(flint, oracle):
    # gemm_fp8_cutlass_test.cc:248-283
    row = [0x00, 0x7e, 0xfe, 0x38, 0xb8, 0x3c, 0x40, 0x44, 0x48, 0x4c, 0x50, 0x54, 0x58, 0x5c, 0x60, 0x64,
           0x68, 0x6c, 0x70, 0x74, 0x78, 0x7c, 0x7d, 0x7a, 0xf8, 0xb0, 0x30, 0x28, 0x20, 0xec, 0x76, 0xc4]
    codes = np.tile(np.array(row, np.uint8), (8, 1))
    row_sum = np.float32(sum(float(oracle.e4m3_decode_table()[c]) for c in row))
    a = f16(np.ones((4, 32)))
    for scale in (0.001953125, 3.0, 0.0):
        got = from_f16(run(flint, a, codes, scale))
        assert np.all(np.isfinite(got))
        want = row_sum * np.float32(scale)
        assert np.all(np.abs(got - want) <= abs(want) * 1e-3), (scale, got[0], want)


@pytest.mark.parametrize("m", [3, 600])
def test_addend_rounds_once(flint, m):
    # gemm_fp8_cutlass_test.cc:304-332
    n, k = 136, 32
    codes = np.full((n, k), 0x38, np.uint8)
    rows = np.zeros((m, k), np.float32)
    rows[:, 0], rows[:, 1] = 2048.0, 1.0
    a = f16(rows)
    for addend in (f16(np.ones(n)), f16(np.ones((m, n)))):
        for expand in (False, True):
            got = from_f16(run(flint, a, codes, 1.0, addend, expand=expand))
            assert np.all(got == 2050.0)
    plain = from_f16(run(flint, a, codes, 1.0))
    assert np.all(plain == 2048.0)


@pytest.mark.parametrize("shape_a", [(7, 64), (600, 64), (3, 5, 64)])
def test_addend_agrees_with_product_and_add(flint, oracle, shape_a):
    # gemm_fp8_cutlass_test.cc:334-361, including the addend broadcast over a leading dimension.
    rng = np.random.default_rng(13 + len(shape_a))
    n = 40
    codes = random_codes(rng, n, 64)
    a = f16(rng.standard_normal(shape_a))
    out_shape = shape_a[:-1] + (n,)
    addends = [(n,), out_shape]
    if len(out_shape) > 2:
        addends.append((1, out_shape[1], n))
    for ashape in addends:
        addend = f16(rng.standard_normal(ashape))
        for expand in (False, True):
            got = run(flint, a, codes, K_SCALE, addend, expand=expand)
            want = oracle.fp8_matmul(a, codes, [K_SCALE], addend)
            check_parity(oracle, got, want, False, rel=2e-3, what=f"{shape_a}+{ashape}")


def test_in_place_residual(flint):
    # flint/metal_native/operators_test.cc:1474-1477: out may be the residual itself.
    F = flint
    m, n, k = 130, 136, 32
    codes = np.zeros((n, k), np.uint8)
    codes[:, 0], codes[:, 1] = 0x78, 0x20
    a = np.zeros((m, k), np.float32)
    a[:, 0] = a[:, 1] = 1.0
    res = dev(F, f16(np.ones((m, n))), F.DType.FLOAT16)
    ad, wd, sd = dev(F, f16(a), F.DType.FLOAT16), dev(F, codes, F.DType.FP8E4M3), dev(F, np.array([8.0], np.float32), F.DType.FLOAT)
    F.check(F.lib().fl_fp8_matmul_add(ad.raw(), wd.raw(), sd.raw(), res.raw(), res.raw()))
    assert np.all(from_f16(res.numpy()) == 2050.0)


def test_exact_values_and_refusals_on_the_card(flint, oracle):
    # waifu/tests/tensor_cuda.rs:341-416 and flint/capi_test.cc:448-487
    F = flint
    values = np.array([448.0, -224.0, 112.0, 56.0, 28.0, 14.0, 7.0, 3.5, 1.75, 0.875, 0.0, -1.0, 2.0, -4.0, 8.0, -16.0], np.float32)
    row = np.array([0x7e, 0xf6, 0x6e, 0x66, 0x5e, 0x56, 0x4e, 0x46, 0x3e, 0x36, 0x00, 0xb8, 0x40, 0xc8, 0x50, 0xd8], np.uint8)
    codes = np.tile(row, (8, 1))
    ramp = (np.arange(16, dtype=np.float32) - 8.0) / 4.0
    a_np = np.stack([np.ones(16, np.float32), ramp])
    a = dev(F, f16(a_np), F.DType.FLOAT16)
    w = dev(F, codes, F.DType.FP8E4M3)
    s = dev(F, np.array([K_SCALE], np.float32), F.DType.FLOAT)
    got = from_f16(F.fp8_matmul(a, w, s).numpy())
    for m in range(2):
        want = np.float32(np.sum(a_np[m] * values, dtype=np.float32) * K_SCALE)
        assert np.all(np.abs(got[m] - want) <= abs(want) * 1e-3)
    with pytest.raises(F.FlintError) as e:
        F.fp8_matmul(a, w, dev(F, np.full(8, K_SCALE, np.float32), F.DType.FLOAT))
    assert e.value.code == F.FL_ERROR_INVALID_ARG
    with pytest.raises(F.FlintError):  # a scale on the host
        F.fp8_matmul(a, w, F.Tensor.from_numpy(np.array([K_SCALE], np.float32), F.DType.FLOAT, F.Device.CPU))
    with pytest.raises(F.FlintError):  # rows not a multiple of 8
        F.fp8_matmul(a, dev(F, codes[:7], F.DType.FP8E4M3), s)
    with pytest.raises(F.FlintError):  # k not a multiple of 16
        F.fp8_matmul(dev(F, f16(a_np[:, :8]), F.DType.FLOAT16), dev(F, codes[:, :8], F.DType.FP8E4M3), s)
    with pytest.raises(F.FlintError):  # an addend that does not broadcast
        F.fp8_matmul_add(a, w, s, dev(F, f16(np.zeros(3)), F.DType.FLOAT16))
    # all-ones weight, scale 0.5: exactly 8 (waifu/tests/foundation.rs:311-349)
    y = from_f16(F.fp8_matmul(dev(F, f16(np.ones((1, 16))), F.DType.FLOAT16), dev(F, np.full((8, 16), 0x38, np.uint8), F.DType.FP8E4M3),
                              dev(F, np.array([0.5], np.float32), F.DType.FLOAT)).numpy())
    assert np.array_equal(y, np.full((1, 8), 8.0, np.float32))


def test_misaligned_view_offset(flint, oracle):
    """A view may start at any element (flint/capi.h:217-231); the reference only checks
    contiguity, so a base that is not 16-byte aligned has to work too."""
    F = flint
    rng = np.random.default_rng(14)
    m, n, k = 33, 72, 48
    a = f16(rng.standard_normal((m, k)))
    codes = random_codes(rng, n, k)
    pad = 3
    a_buf = dev(F, np.concatenate([np.zeros(pad, np.uint16), a.ravel()]), F.DType.FLOAT16)
    out_buf = F.Tensor.empty((m * n + pad,), F.DType.FLOAT16)
    a_view = a_buf.view_as((m, k), (k, 1), pad)
    out_view = out_buf.view_as((m, n), (n, 1), pad)
    wd, sd = dev(F, codes, F.DType.FP8E4M3), dev(F, np.array([K_SCALE], np.float32), F.DType.FLOAT)
    F.check(F.lib().fl_fp8_matmul(a_view.raw(), wd.raw(), sd.raw(), out_view.raw()))
    got = out_buf.numpy()[pad:].reshape(m, n)
    check_parity(oracle, got, oracle.fp8_matmul(a, codes, [K_SCALE]), False, what="offset view")


@pytest.mark.parametrize("name", ["matmul_a", "matmul_b", "matmul_c"])
def test_golden_vectors(flint, oracle, name):
    fx = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantized_linear.npz"))
    addend = fx[name + "_addend"] if name + "_addend" in fx else None
    got = run(flint, fx[name + "_a"], fx[name + "_codes"], fx[name + "_scale"], addend)
    check_parity(oracle, got, fx[name + "_y"], False, what=name)


def test_bf16_variant(flint, oracle):
    rng = np.random.default_rng(15)
    m, n, k = 200, 264, 160
    a = oracle.narrow(rng.standard_normal((m, k)).astype(np.float32), True)
    codes = random_codes(rng, n, k)
    bias = oracle.narrow(rng.standard_normal(n).astype(np.float32), True)
    got = run(flint, a, codes, K_SCALE, bias, dtype=flint.DType.BFLOAT16)
    check_parity(oracle, got, oracle.fp8_matmul(a, codes, [K_SCALE], bias, is_bf16=True), True, what="bf16")


# (half rows against wide weights, k a multiple of 64, run with the weight on the tensor cores' M
# side: the first shape and the last fourteen, among them ragged last tiles of channels, last stages
# with one, two and three of their four blocks, more CTAs than the GPU has SMs, and 17 to 64 rows,
# which the instruction takes as N = 32 or 64)
@pytest.mark.parametrize("m,n,k,bf16", [(1, 16384, 3072, False), (16, 264, 3072, True), (9, 72, 12288, False),
                                        (5, 4096, 80, True), (2, 64, 4112, False), (7, 72, 6160, True), (3, 136, 1040, False),
                                        (16, 12288, 64, False), (11, 12296, 4160, False), (4, 18432, 3072, False), (8, 8200, 320, False),
                                        (1, 8192, 2240, False), (2, 6144, 2112, False), (8, 3080, 2176, False), (16, 24576, 2048, False),
                                        (17, 8200, 2112, False), (32, 3072, 4096, False), (25, 24576, 2048, False),
                                        (33, 3080, 2112, False), (64, 8192, 2048, False), (48, 24576, 2048, False)])
def test_few_rows(flint, oracle, m, n, k, bf16):
    """Few rows take one-launch paths that widen the weight in registers (against wide weights:
    into tensor memory, up to 64 rows); the first shape is the reference's decode benchmark
    (docs/fp8.md:225-244)."""
    rng = np.random.default_rng(16 + m + n + k)
    a = oracle.narrow(rng.standard_normal((m, k)).astype(np.float32), bf16)
    codes = random_codes(rng, n, k)
    dtype = flint.DType.BFLOAT16 if bf16 else flint.DType.FLOAT16
    want = oracle.fp8_matmul(a, codes, [K_SCALE], is_bf16=bf16)
    check_parity(oracle, run(flint, a, codes, K_SCALE, dtype=dtype), want, bf16, what=f"few rows {m}x{n}x{k}")
    for ashape in ((n,), (m, n)):
        addend = oracle.narrow(rng.standard_normal(ashape).astype(np.float32), bf16)
        got = run(flint, a, codes, K_SCALE, addend, dtype=dtype, expand=False)
        want = oracle.fp8_matmul(a, codes, [K_SCALE], addend, is_bf16=bf16)
        check_parity(oracle, got, want, bf16, what=f"few rows {m}x{n}x{k}+{ashape}")


def test_few_rows_in_place_residual(flint):
    F = flint
    m, n, k = 4, 136, 32
    codes = np.zeros((n, k), np.uint8)
    codes[:, 0], codes[:, 1] = 0x78, 0x20
    a = np.zeros((m, k), np.float32)
    a[:, 0] = a[:, 1] = 1.0
    res = dev(F, f16(np.ones((m, n))), F.DType.FLOAT16)
    ad, wd, sd = dev(F, f16(a), F.DType.FLOAT16), dev(F, codes, F.DType.FP8E4M3), dev(F, np.array([8.0], np.float32), F.DType.FLOAT)
    F.check(F.lib().fl_fp8_matmul_add(ad.raw(), wd.raw(), sd.raw(), res.raw(), res.raw()))
    assert np.all(from_f16(res.numpy()) == 2050.0)
