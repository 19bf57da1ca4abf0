"""Generates tests/golden/block_steps.npz: outputs of the reference's own CPU operators for the
steps either side of a projection (fl_layer_norm without affine, fl_rms_norm, fl_swiglu;
flint/cpu/normalizations.cc, flint/cpu/glu.cc) on seeded bfloat16 inputs, computed through
oracle/_ref/libflint_cpu.so on the widened inputs and narrowed to bfloat16. Run where the
reference checkout exists and oracle/_ref has been built (`make -C oracle ref`):

    python tests/golden/make_block_steps.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "block_steps.npz")


def main():
    assert O.have_ref(), "build oracle/_ref first (make -C oracle ref)"
    rng = np.random.default_rng(20240611)
    R = O.ref()
    fx = {}
    x = O.narrow((rng.standard_normal((24, 1040)) * 1.7 + 0.3).astype(np.float32), True)
    fx["ln_x"], fx["ln_eps"] = x, np.array([1e-6], np.float32)
    fx["ln_y"] = O.narrow(R.layer_norm(O.widen(x, True), 1e-6), True)
    heads, head_dim, rows = 2, 128, 10
    qkv = O.narrow((rng.standard_normal((rows, 3 * heads * head_dim)) * 2).astype(np.float32), True)
    w = O.narrow((1.0 + 0.1 * rng.standard_normal(head_dim)).astype(np.float32), True)
    qk = O.widen(qkv[:, :2 * heads * head_dim], True).reshape(rows * 2 * heads, head_dim)
    fx["rms_qkv"], fx["rms_w"], fx["rms_heads"] = qkv, w, np.array([heads], np.int32)
    fx["rms_y"] = O.narrow(R.rms_norm(qk, O.widen(w, True), 1e-6), True).reshape(rows, 2 * heads * head_dim)
    g = O.narrow((rng.standard_normal((12, 2 * 520)) * 3).astype(np.float32), True)
    fx["swiglu_x"] = g
    fx["swiglu_y"] = O.narrow(R.swiglu(O.widen(g, True)), True)
    np.savez_compressed(OUT, **fx)
    print("wrote", OUT, {k: v.shape for k, v in fx.items()})


if __name__ == "__main__":
    main()
