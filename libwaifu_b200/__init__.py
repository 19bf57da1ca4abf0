"""flint-sm100: a B200 (sm_100a) implementation of flint's quantized matmul/linear path.

``libwaifu_b200.flint`` is the host-side mirror of the reference's wrapper over the C ABI;
``libwaifu_b200.build`` compiles ``lib/libflint_sm100.so`` from ``csrc/``.
"""
from . import build as build_ext  # noqa: F401

__all__ = ["flint", "build_ext"]
