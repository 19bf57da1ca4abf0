"""Builds libflint_sm100.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libflint_sm100.so")
SOURCES = ["gemm_sm100.cu", "quant_sm100.cu", "skinny_sm100.cu", "block_sm100.cu", "attention_sm100.cu", "elementwise_sm100.cu",
           "selftest_sm100.cu", "matmul_simt_sm100.cu", "peer_sm100.cu", "fewrow_tc_sm100.cu", "flint_capi.cu"]
HEADERS = ["gemm_sm100.cuh", "quant_sm100.cuh", "skinny_sm100.cuh", "block_sm100.cuh", "attention_sm100.cuh", "elementwise_sm100.cuh",
           "selftest_sm100.cuh", "matmul_simt_sm100.cuh", "peer_sm100.cuh", "fewrow_tc_sm100.cuh", "ptx_sm100.cuh", os.path.join("..", "..", "include", "flint_sm100.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "static", "-Wno-deprecated-gpu-targets",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA extension cannot be built")


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link the shared library. Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = _nvcc()
    from concurrent.futures import ThreadPoolExecutor

    def compile_one(src: str) -> str:
        obj = os.path.join(LIB_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    subprocess.run([nvcc, "-shared", "-cudart", "static", "-Wno-deprecated-gpu-targets", "-o", LIB_PATH, *objs, "-lpthread", "-ldl", "-lrt"], check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
