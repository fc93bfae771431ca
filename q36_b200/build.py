"""Builds libq36moe.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python -m q36_b200.build [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libq36moe.so")
SOURCES = ["moe_api.cu", "moe_route.cu", "moe_gemv.cu", "moe_tc.cu", "moe_tc_fused.cu", "moe_ep.cu", "moe_gguf.cu", "moe_block.cu"]
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--shared", "-cudart", "shared", "-ldl",
]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "q36_moe.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    extra = os.environ.get("Q36_NVCC_EXTRA", "").split()      # e.g. -DQ36_TRACE for the kernels' timing trace
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-ccbin", "g++", *[os.path.join(CSRC, s) for s in SOURCES], "-o", LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("nvcc failed building libq36moe.so")
    with open(os.path.join(HERE, "build_ptxas.log"), "w") as f:
        f.write(r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
