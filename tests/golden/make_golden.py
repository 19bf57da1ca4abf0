"""Generates tests/golden/quantized_linear.npz.

Run in a container where the reference checkout exists and oracle/_ref has been built
(`make -C oracle ref`): the float32 products come from the reference's own CPU fl_matmul
(flint/cpu/matmul.cc:306-322) through oracle/_ref/libflint_cpu.so; quantisation and the epilogue
are the restated ones, cross-checked against torch's float8_e4m3fn cast below. The fixture holds
inputs and expected outputs, so tests that use it need neither the reference nor torch.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quantized_linear.npz")


def main():
    import torch
    assert O.have_ref(), "build oracle/_ref first (make -C oracle ref)"
    rng = np.random.default_rng(20240607)
    fx = {}

    # -- the reference-compatible product: fp16 activation, per-tensor scale, optional addend
    for name, (m, n, k), addend in [("matmul_a", (17, 128, 64), None), ("matmul_b", (129, 264, 96), "bias"),
                                    ("matmul_c", (300, 200, 256), "residual")]:
        a = O.narrow(rng.standard_normal((m, k)).astype(np.float32), False)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        codes, scale = O.quantize_fp8_tensor(w)
        ref = torch.from_numpy(w / scale[0]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        assert np.array_equal(ref, codes)
        ad = None
        if addend == "bias":
            ad = O.narrow(rng.standard_normal(n).astype(np.float32), False)
        elif addend == "residual":
            ad = O.narrow(rng.standard_normal((m, n)).astype(np.float32), False)
        y = O.fp8_matmul(a, codes, scale, ad, is_bf16=False, engine="reference")
        fx[name + "_a"], fx[name + "_codes"], fx[name + "_scale"], fx[name + "_y"] = a, codes, scale, y
        if ad is not None:
            fx[name + "_addend"] = ad

    # -- fp8 linear: bf16, per-channel scales, dynamic activation quantisation, fused epilogue
    for name, (m, n, k), act, use_bias, use_res in [("linear_a", (64, 128, 256), 0, True, False),
                                                     ("linear_b", (130, 72, 208), 1, True, True)]:
        x = O.narrow(rng.standard_normal((m, k)).astype(np.float32), True)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        codes, scales = O.quantize_fp8_rows(w)
        bias = O.narrow((rng.standard_normal(n) * 0.01).astype(np.float32), True) if use_bias else None
        res = O.narrow(rng.standard_normal((m, n)).astype(np.float32), True) if use_res else None
        y = O.fp8_linear(x, codes, scales, bias, res, act, is_bf16=True, engine="reference")
        xc, xs = O.quantize_fp8_act(x, True)
        fx[name + "_x"], fx[name + "_codes"], fx[name + "_scales"], fx[name + "_y"] = x, codes, scales, y
        fx[name + "_xcodes"], fx[name + "_xscales"] = xc, xs
        fx[name + "_act"] = np.array([act], np.int32)
        if bias is not None:
            fx[name + "_bias"] = bias
        if res is not None:
            fx[name + "_res"] = res

    # -- nvfp4 linear
    for name, (m, n, k), act in [("nvfp4_a", (64, 128, 256), 0), ("nvfp4_b", (130, 200, 320), 1)]:
        x = O.narrow(rng.standard_normal((m, k)).astype(np.float32), True)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        codes, sf, g = O.quantize_nvfp4_weight(w)
        bias = O.narrow((rng.standard_normal(n) * 0.01).astype(np.float32), True)
        y = O.nvfp4_linear(x, codes, sf, g, bias, None, act, is_bf16=True, engine="reference")
        xc, xsf = O.quantize_nvfp4_act(x, True)
        fx[name + "_x"], fx[name + "_w"], fx[name + "_codes"], fx[name + "_sf"], fx[name + "_g"] = x, w, codes, sf, g
        fx[name + "_bias"], fx[name + "_y"], fx[name + "_act"] = bias, y, np.array([act], np.int32)
        fx[name + "_xcodes"], fx[name + "_xsf"] = xc, xsf

    np.savez_compressed(OUT, **fx)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(fx), "arrays")


if __name__ == "__main__":
    main()
