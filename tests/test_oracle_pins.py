"""Pins the CPU oracle: every golden vector and known-answer test the reference's own tests hold
for the FP8 path, restated against the oracle, plus exhaustive checks of the codecs against
torch / ml_dtypes casts. Runs without a GPU."""
import numpy as np
import pytest

ml_dtypes = pytest.importorskip("ml_dtypes")
torch = pytest.importorskip("torch")


def f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def from_f16(b):
    return np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


# ---- codecs ----------------------------------------------------------------------------------

def test_e4m3_decode_all_codes_matches_reference_formula(oracle):
    # flint/cuda/gemm_fp8_cutlass_test.cc:95-102, restated independently here.
    table = oracle.e4m3_decode_table()
    for code in range(256):
        if (code & 0x7F) == 0x7F:
            assert np.isnan(table[code])
            continue
        sign, e, m = code >> 7, (code >> 3) & 0xF, code & 7
        mag = np.ldexp(float(m), -9) if e == 0 else np.ldexp(1.0 + m / 8.0, e - 7)
        assert table[code] == (-mag if sign else mag)
    t = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(t, nan=7e7), np.nan_to_num(table, nan=7e7))


def test_e4m3_encode_matches_torch_cast_after_clamp(oracle):
    # tools/model_writer.py:170-172: clamp to +-448, then torch's float8_e4m3fn cast.
    rng = np.random.default_rng(1)
    table = oracle.e4m3_decode_table()
    vals = np.sort(np.unique(table[np.isfinite(table)]))
    mid = ((vals[:-1].astype(np.float64) + vals[1:].astype(np.float64)) / 2).astype(np.float32)
    x = np.concatenate([
        vals, mid, np.nextafter(mid, np.float32(1e9)), np.nextafter(mid, np.float32(-1e9)),
        *(rng.standard_normal(4000).astype(np.float32) * s for s in (1e-4, 1e-2, 1.0, 50.0, 400.0)),
        np.array([448, 449, 463.9, 464, 480, 1e9, -1e9, 0.0, -0.0, 2 ** -10, 2 ** -9, 1.5 * 2 ** -9], dtype=np.float32),
    ]).astype(np.float32)
    mine = oracle.e4m3_encode(x)
    ref = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, ref)
    assert oracle.lib().fo_e4m3_encode(float("nan")) == 0x7F


def test_e2m1_codec_matches_ml_dtypes(oracle):
    rng = np.random.default_rng(2)
    L = oracle.lib()
    assert [L.fo_e2m1_decode(c) for c in range(8)] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert [L.fo_e2m1_decode(c | 8) for c in range(1, 8)] == [-0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    z = np.concatenate([rng.standard_normal(5000).astype(np.float32) * 3,
                        np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -2.5, -5, 6, 7, 100, 0], dtype=np.float32)])
    want = np.clip(z, -6, 6).astype(ml_dtypes.float4_e2m1fn).view(np.uint8) & 0xF
    assert np.array_equal(oracle.e2m1_encode(z), want)


def test_bf16_rounding_known_answers(oracle):
    # waifu/src/qwen_image/pipeline.rs:1080-1094
    L = oracle.lib()
    r = lambda v: L.fo_bf16_to_f32(L.fo_bf16_from_f32(v))
    assert r(1.0) == 1.0
    assert r(987.3) == 988.0
    assert r(985.9) == 984.0
    assert r(986.0) == 984.0  # tie to the even mantissa


def test_16bit_narrowing_matches_torch_and_numpy(oracle):
    rng = np.random.default_rng(3)
    L = oracle.lib()
    y = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-7, 1e-3, 1.0, 3e4)])
    bf = np.array([L.fo_bf16_from_f32(float(v)) for v in y], dtype=np.uint16)
    assert np.array_equal(bf, torch.from_numpy(y).bfloat16().view(torch.uint16).numpy())
    assert np.array_equal(bf, oracle.narrow(y, True))
    assert np.array_equal(bf, oracle.narrow_numpy(y, True))
    with np.errstate(over="ignore"):
        h = y.astype(np.float16).view(np.uint16)
    assert np.array_equal(h, oracle.narrow(y, False))
    assert np.array_equal(np.array([L.fo_f16_from_f32(float(v)) for v in y], dtype=np.uint16), h)
    back = np.array([L.fo_f16_to_f32(int(v)) for v in h[:5000]], dtype=np.float32)
    assert np.array_equal(back, h[:5000].view(np.float16).astype(np.float32))


# ---- the reference's quantizer ------------------------------------------------------------------

def test_per_tensor_quantizer_matches_the_reference_recipe(oracle):
    # tools/model_writer.py:143-174 run with torch, against the oracle's restatement.
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 96, generator=g) * 0.02
    scale = w.abs().amax() / 448.0
    data = (w / scale).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    codes, s = oracle.quantize_fp8_tensor(w.numpy())
    assert np.array_equal(codes, data)
    assert s[0] == np.float32(scale.item())
    # the largest element lands on the top of the range
    assert 0x7E in (codes & 0x7F)
    # an all-zero tensor: scale 0, codes 0, no NaN
    codes, s = oracle.quantize_fp8_tensor(np.zeros((8, 16), np.float32))
    assert s[0] == 0.0 and not codes.any()


def test_per_row_quantizer_is_the_tensor_rule_row_by_row(oracle):
    rng = np.random.default_rng(4)
    w = rng.standard_normal((24, 64)).astype(np.float32) * 0.02
    w[5] = 0.0
    codes, scales = oracle.quantize_fp8_rows(w)
    for r in range(24):
        c, s = oracle.quantize_fp8_tensor(w[r:r + 1])
        assert np.array_equal(c[0], codes[r]) and s[0] == scales[r]
    assert scales[5] == 0.0 and not codes[5].any()


# ---- known-answer tests of the product ------------------------------------------------------------

ROW32 = [0x00, 0x7e, 0xfe, 0x38, 0xb8, 0x3c, 0x40, 0x44, 0x48, 0x4c, 0x50, 0x54, 0x58, 0x5c, 0x60, 0x64,
         0x68, 0x6c, 0x70, 0x74, 0x78, 0x7c, 0x7d, 0x7a, 0xf8, 0xb0, 0x30, 0x28, 0x20, 0xec, 0x76, 0xc4]


@pytest.mark.parametrize("engine", ["port", "reference"])
def test_scale_applied_known_answer(oracle, engine):
    # flint/cuda/gemm_fp8_cutlass_test.cc:248-283
    if engine == "reference" and not oracle.have_ref():
        pytest.skip("reference CPU build not present")
    codes = np.tile(np.array(ROW32, dtype=np.uint8), (8, 1))
    table = oracle.e4m3_decode_table()
    row_sum = np.float32(0)
    for c in ROW32:
        row_sum = np.float32(row_sum + table[c])
    assert row_sum != 0
    a = f16(np.ones((4, 32)))
    for scale in (0.001953125, 3.0, 0.0):
        out = from_f16(oracle.fp8_matmul(a, codes, np.array([scale], np.float32), engine=engine))
        assert np.all(np.isfinite(out))
        want = row_sum * np.float32(scale)
        assert np.all(np.abs(out - want) <= abs(want) * 1e-3)


@pytest.mark.parametrize("m", [3, 600])
def test_addend_rounds_once_known_answer(oracle, m):
    # flint/cuda/gemm_fp8_cutlass_test.cc:304-332: 2048 + 1 (+ 1) in half.
    n, k = 136, 32
    codes = np.full((n, k), 0x38, dtype=np.uint8)
    rows = np.zeros((m, k), np.float32)
    rows[:, 0] = 2048.0
    rows[:, 1] = 1.0
    a = f16(rows)
    one = np.array([1.0], np.float32)
    for addend in (f16(np.ones(n)), f16(np.ones((m, n)))):
        assert np.all(from_f16(oracle.fp8_matmul(a, codes, one, addend)) == 2050.0)
    twice = from_f16(oracle.fp8_matmul(a, codes, one)) + 1.0
    assert np.all(twice.astype(np.float16) == 2048.0)


def test_metal_rounds_once_known_answer(oracle):
    # flint/metal_native/operators_test.cc:1443-1478: codes 0x78 (256) and 0x20 (0.125), scale 8.
    for k in (32, 40):
        for m in (1, 3, 130):
            codes = np.zeros((136, k), np.uint8)
            codes[:, 0], codes[:, 1] = 0x78, 0x20
            a = np.zeros((m, k), np.float32)
            a[:, 0] = a[:, 1] = 1.0
            s = np.array([8.0], np.float32)
            assert np.all(from_f16(oracle.fp8_matmul(f16(a), codes, s, f16(np.ones(136)))) == 2050.0)
            assert np.all(from_f16(oracle.fp8_matmul(f16(a), codes, s)) == 2048.0)


def test_exact_values_known_answer(oracle):
    # waifu/tests/tensor_cuda.rs:352-392
    values = np.array([448.0, -224.0, 112.0, 56.0, 28.0, 14.0, 7.0, 3.5, 1.75, 0.875, 0.0, -1.0, 2.0, -4.0, 8.0, -16.0], np.float32)
    codes_row = np.array([0x7e, 0xf6, 0x6e, 0x66, 0x5e, 0x56, 0x4e, 0x46, 0x3e, 0x36, 0x00, 0xb8, 0x40, 0xc8, 0x50, 0xd8], np.uint8)
    assert np.array_equal(oracle.e4m3_decode_table()[codes_row], values)
    assert np.array_equal(oracle.e4m3_encode(values), codes_row)
    scale = np.float32(0.0137)
    ramp = (np.arange(16, dtype=np.float32) - 8.0) / 4.0
    a = np.stack([np.ones(16, np.float32), ramp])
    out = from_f16(oracle.fp8_matmul(f16(a), np.tile(codes_row, (8, 1)), np.array([scale])))
    for m in range(2):
        want = np.float32(np.sum(a[m] * values, dtype=np.float32) * scale)
        assert np.all(np.abs(out[m] - want) <= abs(want) * 1e-3)


def test_all_ones_weight_known_answer(oracle):
    # waifu/tests/foundation.rs:311-349: sixteen 1.0 codes, scale 0.5 -> exactly 8.
    out = from_f16(oracle.fp8_matmul(f16(np.ones((1, 16))), np.full((8, 16), 0x38, np.uint8), np.array([0.5], np.float32)))
    assert np.array_equal(out, np.full((1, 8), 8.0, np.float32))


def test_port_gemm_agrees_with_reference_gemm(oracle):
    if not oracle.have_ref():
        pytest.skip("reference CPU build not present")
    rng = np.random.default_rng(5)
    for (m, n, k) in [(1, 8, 16), (17, 128, 64), (129, 264, 96), (300, 200, 256)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((n, k)).astype(np.float32)
        exact = oracle.gemm_f64_nt(a, b)
        assert oracle.rel_l2(oracle.gemm_f32_nt(a, b, "reference"), exact) < 2e-6
        assert oracle.rel_l2(oracle.gemm_f32_nt(a, b, "port"), exact) < 2e-6


def test_gelu_tanh_epilogue_matches_torch(oracle):
    rng = np.random.default_rng(6)
    acc = rng.standard_normal((16, 32)).astype(np.float32) * 3
    got = oracle.widen(oracle.epilogue(acc, act=oracle.ACT_GELU_TANH, out_is_bf16=True), True)
    want = torch.nn.functional.gelu(torch.from_numpy(acc), approximate="tanh").bfloat16().float().numpy()
    assert np.max(np.abs(got - want)) <= np.max(np.abs(want)) * 2 ** -8


def test_nvfp4_quantizer_roundtrip_properties(oracle):
    rng = np.random.default_rng(7)
    w = rng.standard_normal((16, 64)).astype(np.float32) * 0.02
    w[3, 16:32] = 0.0
    codes, sf, g = oracle.quantize_nvfp4_weight(w)
    assert g[0] == np.float32(np.max(np.abs(w)) / np.float32(448.0 * 6.0))
    assert sf[3, 1] == 0 and not codes[3, 8:16].any()
    assert not ((sf & 0x80).any())  # unsigned scales
    deq = oracle.decode_nvfp4(codes, sf) * g[0]
    # e2m1 with a fitted block scale: at most half a step of the coarsest spacing (2 of 6)
    # relative to the block amax, plus the e4m3 rounding of the block scale.
    blocks_w = w.reshape(16, 4, 16)
    blocks_d = deq.reshape(16, 4, 16)
    amax = np.max(np.abs(blocks_w), axis=2, keepdims=True)
    assert np.all(np.abs(blocks_d - blocks_w) <= amax * (1.0 / 6.0 + 0.07) + 1e-12)


# ---- the block-step restatements against the reference's own CPU operators ----------------------

def _needs_ref(oracle):
    if not oracle.have_ref():
        pytest.skip("the reference's CPU build is not present")


def test_layernorm_restatement_against_the_reference_operator(oracle):
    """layernorm_modulate with no scale and shift is the reference's fl_layer_norm narrowed to 16
    bits. The reference sums in float32 in row order and the restatement in float64, so a value on
    a 16-bit rounding boundary may fall either way: at most one step, nearly all identical."""
    _needs_ref(oracle)
    rng = np.random.default_rng(101)
    for k in (16, 1040, 3072):
        x16 = oracle.narrow((rng.standard_normal((33, k)) * 1.7 + 0.3).astype(np.float32), True)
        want = oracle.narrow(oracle.ref().layer_norm(oracle.widen(x16, True), 1e-6), True)
        got = oracle.layernorm_modulate(x16, None, None, 1e-6, True)
        assert np.mean(got == want) >= 0.995
        g, w = oracle.widen(got, True), oracle.widen(want, True)
        assert np.all(np.abs(g - w) <= np.maximum(np.abs(w), 2.0 ** -14) * 2.0 ** -7 * 1.01)
    # a constant row: the variance is zero or a rounding residue, eps carries the root
    x16 = oracle.narrow(np.full((2, 64), 3.0, np.float32), True)
    assert not oracle.widen(oracle.layernorm_modulate(x16, None, None, 1e-6, True), True).any()
    assert not oracle.ref().layer_norm(oracle.widen(x16, True), 1e-6).any()


def test_rms_norm_restatement_against_the_reference_operator(oracle):
    """qk_norm_rope with cos = 1, sin = 0 is the reference's fl_rms_norm per head, narrowed (the
    restatement multiplies by one reciprocal per head where the reference divides per element)."""
    _needs_ref(oracle)
    rng = np.random.default_rng(102)
    heads, head_dim, rows = 3, 128, 20
    qkv = oracle.narrow((rng.standard_normal((rows, 3 * heads * head_dim)) * 2).astype(np.float32), True)
    w = oracle.narrow((1.0 + 0.1 * rng.standard_normal(head_dim)).astype(np.float32), True)
    ones, zeros = np.ones((5, head_dim // 2), np.float32), np.zeros((5, head_dim // 2), np.float32)
    got = oracle.qk_norm_rope(qkv, ones, zeros, heads, 1e-6, True, w, w)
    x = oracle.widen(qkv[:, :2 * heads * head_dim], True).reshape(rows * 2 * heads, head_dim)
    want = oracle.narrow(oracle.ref().rms_norm(x, oracle.widen(w, True), 1e-6), True).reshape(rows, 2 * heads * head_dim)
    assert np.array_equal(got[:, 2 * heads * head_dim:], qkv[:, 2 * heads * head_dim:])
    assert np.mean(got[:, :2 * heads * head_dim] == want) >= 0.99
    g, r = oracle.widen(got[:, :2 * heads * head_dim], True), oracle.widen(want, True)
    assert np.all(np.abs(g - r) <= np.maximum(np.abs(r), 2.0 ** -14) * 2.0 ** -7 * 1.01)


def test_swiglu_restatement_against_the_reference_operator(oracle):
    _needs_ref(oracle)
    rng = np.random.default_rng(103)
    x16 = oracle.narrow((rng.standard_normal((17, 2 * 520)) * 3).astype(np.float32), True)
    want = oracle.narrow(oracle.ref().swiglu(oracle.widen(x16, True)), True)
    got = oracle.swiglu(x16, True)
    assert np.mean(got == want) >= 0.995
    g, w = oracle.widen(got, True), oracle.widen(want, True)
    assert np.all(np.abs(g - w) <= np.maximum(np.abs(w), 2.0 ** -14) * 2.0 ** -7 * 1.01)


def test_reciprocal_form_of_the_activation_quantiser_against_the_exporters_division(oracle):
    """The dynamic activation quantiser multiplies by one reciprocal per row where the exporter's
    rule (tools/model_writer.py:164-174) divides every element by the scale. The reference never
    narrows an activation, so nothing of its own pins this choice; this states how far the two
    forms are apart on the benchmark's distribution. The scales are identical. The codes differ only
    at exact ties: where x / s is exactly the midpoint of two codes (which bf16 inputs and a scale
    with few significant bits produce), the division rounds the tie to even and the product with the
    rounded reciprocal, one float32 step above or below the midpoint, rounds to the nearer code. On
    this sample that is about one code in a thousand, all in the few rows whose scale makes ties,
    each by one code step; a product taken with either set of codes agrees to within the path's
    own tolerance. Both are correct roundings of x / s to within half a step plus one float32 ulp."""
    rng = np.random.default_rng(99)
    m, k = 256, 3072
    x16 = oracle.narrow(rng.standard_normal((m, k)).astype(np.float32), True)
    x = oracle.widen(x16, True)
    codes, scales = oracle.quantize_fp8_act(x16, True)
    amax = np.abs(x).max(axis=1)
    s = (amax / np.float32(448.0)).astype(np.float32)
    assert np.array_equal(scales, s)
    encode = oracle.lib().fo_e4m3_encode
    rows = range(0, m, 16)
    quotient = np.stack([(x[r] / s[r]).astype(np.float32) for r in rows])
    div = np.array([[encode(float(v)) for v in row] for row in quotient], np.uint8)
    rec = codes[0:m:16]
    differ = div != rec
    frac = differ.mean()
    assert 0 < frac <= 2e-3, f"{frac:.2e} of the codes differ between the two forms"
    # where they differ it is by one step of the code, never more (sign-magnitude codes of one sign) ...
    assert np.all(np.abs(div[differ].astype(np.int16) - rec[differ].astype(np.int16)) == 1)
    # ... and only at exact ties: the quotient has at most five significant bits there
    tie = quotient[differ].astype(np.float64)
    mant, _ = np.frexp(np.abs(tie))
    assert np.all(mant * 32 == np.floor(mant * 32)), "a code differs away from an exact tie"
    # a product taken with either set of codes is the same to within the path's tolerance
    w = (rng.standard_normal((64, k)) * 0.02).astype(np.float32)
    a = oracle.decode_e4m3(div).astype(np.float64) @ w.T.astype(np.float64)
    b = oracle.decode_e4m3(rec).astype(np.float64) @ w.T.astype(np.float64)
    assert oracle.rel_l2(a, b) <= 5e-3
    print(f"reciprocal vs division: {int(differ.sum())} of {differ.size} codes differ ({frac:.2e})")
