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

# name: (batch, heads, kv_heads, q_len, kv_len, head_dim, mask, is_bf16[, block_size]); the mask is
# flint/capi.h:118-133's number (False/True for none/causal). New cases go at the end, so that
# the random stream of the earlier ones stays what it was.
CASES = {
    "causal_gqa": (1, 4, 2, 96, 130, 64, True, True),
    "full_d128": (2, 2, 2, 70, 70, 128, False, False),
    "block_causal": (1, 2, 1, 150, 200, 64, 2, True, 48),
    "block_diagonal": (1, 2, 2, 300, 300, 128, 3, False, 80),
}


def reference_attention(R, q, k, v, mask, block):
    """The reference's CPU fl_attention. Its CPU device makes no block mask (flint/operators.cc:600-625
    refuses), so under a block mask the rows of one block of positions -- which all see the same keys,
    flint/cuda/attention.cu:165-179 -- go through the reference with no mask over exactly those keys."""
    if mask in (0, 1, False, True):
        return R.attention(q, k, v, mask)
    L, S = q.shape[2], k.shape[2]
    out = np.empty(q.shape, np.float32)
    pos = np.arange(L) + (S - L)
    for b in np.unique(pos // block):
        rows = np.nonzero(pos // block == b)[0]
        first = b * block if mask == 3 else 0
        last = min(S - 1, b * block + block - 1)
        out[:, :, rows] = R.attention(q[:, :, rows], k[:, :, first:last + 1], v[:, :, first:last + 1], False)
    return out


def main():
    assert O.have_ref(), "build oracle/_ref first (make -C oracle ref)"
    rng = np.random.default_rng(20240702)
    R = O.ref()
    fx = {}
    for name, case in CASES.items():
        n, h, hk, L, S, d, causal, is_bf16 = case[:8]
        block = case[8] if len(case) > 8 else 0
        q = O.narrow(rng.standard_normal((n, h, L, d)).astype(np.float32), is_bf16)
        k = O.narrow(rng.standard_normal((n, hk, S, d)).astype(np.float32), is_bf16)
        v = O.narrow(rng.standard_normal((n, hk, S, d)).astype(np.float32), is_bf16)
        fx[name + "_q"], fx[name + "_k"], fx[name + "_v"] = q, k, v
        fx[name + "_flags"] = np.array([int(causal), int(is_bf16), block], np.int32)
        fx[name + "_y"] = reference_attention(R, O.widen(q, is_bf16), O.widen(k, is_bf16), O.widen(v, is_bf16), causal, block)
    np.savez_compressed(OUT, **fx)
    print("wrote", OUT, {k: v.shape for k, v in fx.items()})


if __name__ == "__main__":
    main()
