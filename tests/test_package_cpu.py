"""The package format module on the CPU: the safetensors container against the safetensors
library, the pairing rules against the reference reader's (waifu/src/tensor_file.rs:283-336), and
the exporter's quantisers bit for bit against the oracle and against torch's float8 cast
(tools/model_writer.py:164-174)."""
import numpy as np
import pytest

from libwaifu_b200 import package as P


def randn(rng, shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


def test_e4m3_codes_match_torch_and_the_oracle(oracle):
    import torch
    rng = np.random.default_rng(81)
    x = np.concatenate([randn(rng, 20000, 100.0), randn(rng, 20000, 0.01), np.linspace(-500, 500, 4001, dtype=np.float32),
                        np.array([0.0, -0.0, 448.0, 464.0, 465.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 2.0 ** -6], np.float32)])
    got = P._e4m3_codes(x)
    want = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got, want)
    assert np.array_equal(got, oracle.e4m3_encode(x))
    # every midpoint between neighbouring codes rounds to the even one
    table = P.e4m3_values()
    pos = np.arange(0, 0x7e)
    mids = ((table[pos].astype(np.float64) + table[pos + 1]) / 2).astype(np.float32)
    assert np.array_equal(P._e4m3_codes(mids), torch.from_numpy(mids).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    assert np.array_equal(table[:0x7f], oracle.e4m3_decode_table()[:0x7f])


def test_quantisers_match_the_oracle_bit_for_bit(oracle):
    rng = np.random.default_rng(82)
    w = randn(rng, (72, 208), 0.02)
    w[5] = 0
    w[9, 3] = 7.5
    codes, scales = P.quantize_fp8_row_scale(w)
    want_c, want_s = oracle.quantize_fp8_rows(w)
    assert np.array_equal(codes, want_c) and np.array_equal(scales.view(np.uint32), want_s.view(np.uint32))
    codes, scale = P.quantize_fp8_tensor_scale(w)
    want_c, want_s = oracle.quantize_fp8_tensor(w)
    assert np.array_equal(codes, want_c) and np.array_equal(scale.view(np.uint32), np.asarray(want_s, np.float32).reshape(1).view(np.uint32))
    z_codes, z_scale = P.quantize_fp8_tensor_scale(np.zeros((8, 16), np.float32))
    assert not z_codes.any() and z_scale[0] == 0
    packed, block, g = P.quantize_nvfp4(w[:, :192])
    want_p, want_b, want_g = oracle.quantize_nvfp4_weight(w[:, :192])
    assert np.array_equal(g.view(np.uint32), np.asarray(want_g, np.float32).reshape(1).view(np.uint32))
    assert np.array_equal(block, want_b)
    assert np.array_equal(packed, want_p)


def test_container_round_trip_and_the_safetensors_library(tmp_path):
    import torch
    from safetensors.torch import load_file, save_file
    rng = np.random.default_rng(83)
    tensors = {"a.weight": randn(rng, (16, 32), 0.02), "a.bias": randn(rng, (16,)), "b.weight": randn(rng, (8, 64), 0.02)}
    path = str(tmp_path / "m.safetensors")
    P.write_package(path, tensors, ["a.weight", "b.weight"], "fp8_row_scale")
    got, fmt = P.read_package(path)
    assert fmt == "fp8_row_scale"
    assert sorted(got) == ["a.bias", "a.weight", "a.weight.scale", "b.weight", "b.weight.scale"]
    assert got["a.weight"].dtype == "F8_E4M3" and got["a.weight"].shape == (16, 32)
    assert got["a.weight.scale"].dtype == "F32" and got["a.weight.scale"].shape == (16,)
    assert np.array_equal(got["a.bias"].array, tensors["a.bias"])
    # the library reads what this wrote ...
    lib = load_file(path)
    assert lib["a.weight"].dtype == torch.float8_e4m3fn
    assert np.array_equal(lib["a.weight"].view(torch.uint8).numpy(), got["a.weight"].array)
    assert np.array_equal(lib["a.weight.scale"].numpy(), got["a.weight.scale"].array)
    # ... and this reads what the library (the reference exporter's writer) wrote
    ref = str(tmp_path / "ref.safetensors")
    w = torch.from_numpy(tensors["a.weight"])
    scale = w.abs().amax() / 448.0
    save_file({"p.weight": (w / scale).clamp(-448, 448).to(torch.float8_e4m3fn), "p.weight.scale": scale.reshape(1)}, ref,
              metadata={"weight_format": "fp8_tensor_scale"})
    got, fmt = P.read_package(ref)
    assert fmt == "fp8_tensor_scale"
    mine, my_scale = P.quantize_fp8_tensor_scale(tensors["a.weight"])
    assert np.array_equal(got["p.weight"].array, mine) and got["p.weight.scale"].array[0] == my_scale[0]


def test_pairing_rules(tmp_path):
    rng = np.random.default_rng(84)
    w = randn(rng, (16, 32), 0.02)
    codes, row = P.quantize_fp8_row_scale(w)
    _, one = P.quantize_fp8_tensor_scale(w)
    f8 = P.StoredTensor("F8_E4M3", codes)
    with pytest.raises(P.PackageError, match="no 'w.scale' beside it"):
        P.check_pairs({"w": f8}, "fp8_tensor_scale")
    with pytest.raises(P.PackageError, match="scale per row"):  # the reference's refusal of the old per-row format
        P.check_pairs({"w": f8, "w.scale": P.StoredTensor("F32", row)}, "fp8_tensor_scale")
    with pytest.raises(P.PackageError, match="fp8_tensor_scale"):
        P.check_pairs({"w": f8, "w.scale": P.StoredTensor("F32", one)}, "fp8_row_scale")
    with pytest.raises(P.PackageError, match="weight_format is 'float'"):
        P.check_pairs({"w": f8, "w.scale": P.StoredTensor("F32", one)}, "float")
    with pytest.raises(P.PackageError):
        P.check_pairs({"w": f8, "w.scale": P.StoredTensor("F16", one.astype(np.float16))}, "fp8_tensor_scale")
    P.check_pairs({"w": f8, "w.scale": P.StoredTensor("F32", one)}, "fp8_tensor_scale")
    P.check_pairs({"w": f8, "w.scale": P.StoredTensor("F32", row)}, "fp8_row_scale")
    P.check_pairs({"gain.scale": P.StoredTensor("F32", one)}, "float")  # an unlucky name is an ordinary tensor
    packed, block, g = P.quantize_nvfp4(w)
    nv = {"w": P.StoredTensor("U8", packed), "w.block_scale": P.StoredTensor("F8_E4M3", block), "w.scale": P.StoredTensor("F32", g)}
    P.check_pairs(nv, "nvfp4")
    with pytest.raises(P.PackageError):
        P.check_pairs({k: v for k, v in nv.items() if k != "w.scale"}, "nvfp4")
    with pytest.raises(P.PackageError, match="k / 16"):
        P.check_pairs(dict(nv, **{"w.block_scale": P.StoredTensor("F8_E4M3", block[:, :1])}), "nvfp4")
    with pytest.raises(P.PackageError):
        P.check_pairs({}, "fp8")  # no longer a name a manifest may use (docs/fp8.md:113-115)
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!")
    with pytest.raises(P.PackageError, match="not JSON"):
        P.read_safetensors(str(bad))


def test_pairing_rules_catch_mis_named_and_lost_companions(tmp_path):
    """A ".block_scale" name excuses an F8_E4M3 tensor from its ".scale" only in an nvfp4 package, and
    an nvfp4 weight whose block scales or global scale were lost or renamed is caught by name."""
    rng = np.random.default_rng(85)
    w = randn(rng, (16, 32), 0.02)
    codes, row = P.quantize_fp8_row_scale(w)
    f8 = P.StoredTensor("F8_E4M3", codes)
    for fmt in ("fp8_tensor_scale", "fp8_row_scale"):
        with pytest.raises(P.PackageError, match="no 'w.block_scale.scale' beside it"):
            P.check_pairs({"w.block_scale": f8}, fmt)
    packed, block, g = P.quantize_nvfp4(w)
    nv = {"w": P.StoredTensor("U8", packed), "w.block_scale": P.StoredTensor("F8_E4M3", block), "w.scale": P.StoredTensor("F32", g)}
    # the block scales lost: found through the F32[1] scale beside the U8 matrix, and through the list
    lost = {k: v for k, v in nv.items() if k != "w.block_scale"}
    with pytest.raises(P.PackageError, match="no 'w.block_scale' beside it"):
        P.check_pairs(lost, "nvfp4")
    with pytest.raises(P.PackageError, match="no 'w.block_scale' beside it"):
        P.check_pairs({"w": nv["w"]}, "nvfp4", ["w"])
    with pytest.raises(P.PackageError, match="no 'w.scale' beside it"):
        P.check_pairs({k: v for k, v in nv.items() if k != "w.scale"}, "nvfp4", ["w"])
    with pytest.raises(P.PackageError, match="block scales are F8_E4M3"):
        P.check_pairs(dict(nv, **{"w.block_scale": P.StoredTensor("U8", block)}), "nvfp4")
    with pytest.raises(P.PackageError, match="no codes tensor"):
        P.check_pairs({k: v for k, v in nv.items() if k != "w"}, "nvfp4")
    # the written file names its quantized matrices, so a reader notices a companion that went missing
    path = str(tmp_path / "nv.safetensors")
    P.write_package(path, {"w": w, "b": randn(rng, (16,), 0.01)}, ["w"], "nvfp4")
    tensors, fmt = P.read_package(path)
    assert fmt == "nvfp4" and set(tensors) == {"w", "w.block_scale", "w.scale", "b"}
    stored, meta = P.read_safetensors(path)
    del stored["w.block_scale"], stored["w.scale"]
    P.write_safetensors(path, stored, meta)
    with pytest.raises(P.PackageError, match="no 'w.block_scale' beside it"):
        P.read_package(path)
