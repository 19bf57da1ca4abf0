"""A package written by the exporter's arithmetic, read back, uploaded and multiplied on the GPU:
each weight format reaches the entry point that reads it, with the oracle as the checker; and the
device-side quantisers write the same bits as the exporter's."""
import numpy as np
import pytest

from helpers import check_parity, randn
from libwaifu_b200 import package as P

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


@pytest.mark.parametrize("weight_format", ["fp8_tensor_scale", "fp8_row_scale", "nvfp4"])
def test_package_to_product(flint, oracle, tmp_path, weight_format):
    F = flint
    rng = np.random.default_rng(91)
    m, n, k = 96, 136, 256
    w = randn(rng, (n, k), 0.02)
    bias = oracle.narrow(randn(rng, (n,), 0.01), True)
    path = str(tmp_path / "model.safetensors")
    P.write_package(path, {"proj.weight": w, "proj.bias": randn(rng, (n,), 0.01)}, ["proj.weight"], weight_format)
    tensors, fmt = P.read_package(path)
    assert fmt == weight_format
    operands = P.upload_linear(tensors, "proj.weight", fmt)
    x = oracle.narrow(randn(rng, (m, k)), True)
    bf = F.DType.BFLOAT16
    if weight_format == "fp8_tensor_scale":
        # the reference's own format through the reference's own entry point (fp16 activation)
        x16 = oracle.narrow(randn(rng, (m, k)), False)
        got = F.fp8_matmul(dev(F, x16, F.DType.FLOAT16), operands[0], operands[1]).numpy()
        want = oracle.fp8_matmul(x16, tensors["proj.weight"].array, tensors["proj.weight.scale"].array)
        check_parity(oracle, got, want, False, what="package -> fl_fp8_matmul")
        got = F.fp8_linear(dev(F, x, bf), operands[0], operands[1], dev(F, bias, bf), None, 0).numpy()
        want = oracle.fp8_linear(x, tensors["proj.weight"].array, tensors["proj.weight.scale"].array, bias, None, 0, True)
    elif weight_format == "fp8_row_scale":
        got = F.fp8_linear(dev(F, x, bf), operands[0], operands[1], dev(F, bias, bf), None, 0).numpy()
        want = oracle.fp8_linear(x, tensors["proj.weight"].array, tensors["proj.weight.scale"].array, bias, None, 0, True)
    else:
        got = F.nvfp4_linear(dev(F, x, bf), operands[0], operands[1], operands[2], dev(F, bias, bf), None, 0).numpy()
        want = oracle.nvfp4_linear(x, tensors["proj.weight"].array, tensors["proj.weight.block_scale"].array,
                                   tensors["proj.weight.scale"].array, bias, None, 0, True)
    F.synchronize()
    check_parity(oracle, got, want, True, what=f"package ({weight_format}) -> linear")


def test_device_quantisers_write_the_exporters_bits(flint):
    F = flint
    rng = np.random.default_rng(92)
    w = randn(rng, (72, 416), 0.02)
    w[3] = 0
    codes, scales = F.quantize_fp8_rows(dev(F, w, F.DType.FLOAT))
    want_c, want_s = P.quantize_fp8_row_scale(w)
    assert np.array_equal(codes.numpy(), want_c)
    assert np.array_equal(scales.numpy().view(np.uint32), want_s.view(np.uint32))
    packed, block, g = F.quantize_nvfp4(dev(F, w, F.DType.FLOAT))
    want_p, want_b, want_g = P.quantize_nvfp4(w)
    assert np.array_equal(g.numpy().view(np.uint32), want_g.view(np.uint32))
    assert np.array_equal(block.numpy(), want_b)
    assert np.array_equal(packed.numpy(), want_p)
    F.synchronize()
