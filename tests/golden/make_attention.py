"""Generates tests/golden/attention.npz: outputs of the reference's own CPU fl_attention
(flint/capi.h:532-544, flint/operators.cc:148-230) on seeded 16-bit inputs, computed through
oracle/_ref/libflint_cpu.so on the widened inputs and kept as float32. Run where the reference
checkout exists and oracle/_ref has been built (`make -C oracle ref`):

    python tests/golden/make_attention.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention.npz")

# name: (batch, heads, kv_heads, q_len, kv_len, head_dim, causal, is_bf16)
CASES = {
    "causal_gqa": (1, 4, 2, 96, 130, 64, True, True),
    "full_d128": (2, 2, 2, 70, 70, 128, False, False),
}


def main():
    assert O.have_ref(), "build oracle/_ref first (make -C oracle ref)"
    rng = np.random.default_rng(20240702)
    R = O.ref()
    fx = {}
    for name, (n, h, hk, L, S, d, causal, is_bf16) in CASES.items():
        q = O.narrow(rng.standard_normal((n, h, L, d)).astype(np.float32), is_bf16)
        k = O.narrow(rng.standard_normal((n, hk, S, d)).astype(np.float32), is_bf16)
        v = O.narrow(rng.standard_normal((n, hk, S, d)).astype(np.float32), is_bf16)
        fx[name + "_q"], fx[name + "_k"], fx[name + "_v"] = q, k, v
        fx[name + "_flags"] = np.array([int(causal), int(is_bf16)], np.int32)
        fx[name + "_y"] = R.attention(O.widen(q, is_bf16), O.widen(k, is_bf16), O.widen(v, is_bf16), causal)
    np.savez_compressed(OUT, **fx)
    print("wrote", OUT, {k: v.shape for k, v in fx.items()})


if __name__ == "__main__":
    main()
