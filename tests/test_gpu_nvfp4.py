"""GPU parity of fl_nvfp4_linear (dynamic per-16-block e2m1 activation x NVFP4 weight, unsigned
e4m3 block scales, fp32 global scale) against the CPU oracle, through the C ABI. The reference
has no FP4 of any kind, so these cases are pinned by the oracle's restatement only."""
import os

import numpy as np
import pytest

from helpers import check_parity, randn

pytestmark = pytest.mark.gpu


def dev(F, arr, dtype):
    return F.Tensor.from_numpy(arr, dtype, F.Device.CUDA)


def run(F, x, codes, sf, g, bias=None, res=None, act=0):
    bf = F.DType.BFLOAT16
    out = F.nvfp4_linear(dev(F, x, bf), dev(F, codes, F.DType.FP4E2M1X2), dev(F, sf, F.DType.FP8E4M3),
                         dev(F, g, F.DType.FLOAT), dev(F, bias, bf) if bias is not None else None,
                         dev(F, res, bf) if res is not None else None, act)
    y = out.numpy()
    F.synchronize()
    return y


def test_weight_quantiser_is_bit_exact(flint, oracle):
    rng = np.random.default_rng(61)
    w = randn(rng, (72, 320), 0.02)
    w[3, 16:32] = 0
    codes, sf, g = flint.quantize_nvfp4(dev(flint, w, flint.DType.FLOAT))
    wc, wsf, wg = oracle.quantize_nvfp4_weight(w)
    assert g.numpy().view(np.uint32)[0] == wg.view(np.uint32)[0]
    assert np.array_equal(sf.numpy(), wsf)
    assert np.array_equal(codes.numpy(), wc)


def test_unit_scales_exact(flint, oracle):
    """All block scales 1.0 (0x38), global 1, activations already on the e2m1 grid with a block
    amax of 6: every product and sum is exact, so the output must match bit for bit."""
    rng = np.random.default_rng(62)
    m, n, k = 128, 192, 256
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)
    xv = grid[rng.integers(0, 8, size=(m, k))] * rng.choice([-1.0, 1.0], size=(m, k)).astype(np.float32)
    xv[:, ::16] = 6.0
    x = oracle.narrow(xv, True)
    wcodes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    sf = np.full((n, k // 16), 0x38, np.uint8)
    g = np.array([1.0], np.float32)
    got = run(flint, x, wcodes, sf, g)
    want = oracle.nvfp4_linear(x, wcodes, sf, g)
    assert np.array_equal(got, want)


EDGE = [(1, 8, 32), (17, 128, 64), (129, 264, 96), (64, 192, 256), (300, 200, 320), (130, 384, 512),
        (257, 576, 1024), (128, 9216, 256)]


@pytest.mark.parametrize("m,n,k", EDGE)
def test_edge_shapes(flint, oracle, m, n, k):
    rng = np.random.default_rng(200 + m + n + k)
    x = oracle.narrow(randn(rng, (m, k)), True)
    codes, sf, g = oracle.quantize_nvfp4_weight(randn(rng, (n, k), 0.02))
    bias = oracle.narrow(randn(rng, (n,), 0.01), True)
    res = oracle.narrow(randn(rng, (m, n)), True)
    got = run(flint, x, codes, sf, g, bias, res, 0)
    want = oracle.nvfp4_linear(x, codes, sf, g, bias, res, 0)
    check_parity(oracle, got, want, True, what=f"{m}x{n}x{k}")


@pytest.mark.parametrize("name", ["nvfp4_a", "nvfp4_b"])
def test_golden_vectors(flint, oracle, name):
    fx = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantized_linear.npz"))
    got = run(flint, fx[name + "_x"], fx[name + "_codes"], fx[name + "_sf"], fx[name + "_g"], fx[name + "_bias"], None,
              int(fx[name + "_act"][0]))
    check_parity(oracle, got, fx[name + "_y"], True, what=name)


def test_config3_fused_qkv(flint, oracle):
    """X bf16 [4352,3072] ~N(0,1); W [9216,3072] ~N(0,0.02) pre-quantised to NVFP4; bf16 out; seed 0."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(4352, 3072, generator=g).bfloat16().view(torch.uint16).numpy()
    w = (0.02 * torch.randn(9216, 3072, generator=g)).numpy()
    codes, sf, gs = oracle.quantize_nvfp4_weight(w)
    got = run(flint, x, codes, sf, gs)
    want = oracle.nvfp4_linear(x, codes, sf, gs)
    r, u = check_parity(oracle, got, want, True, what="config 3")
    print(f"config 3: rel L2 {r:.3e}, max {u:.2f} ulp")
