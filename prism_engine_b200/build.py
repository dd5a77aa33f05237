"""Builds the sm_100a CUDA library in-tree (``libprism_cuda.so`` / ``.a``).

nvcc cross-compiles without a GPU, so this runs on any box with the CUDA
toolkit.  ``python -m prism_engine_b200.build`` or ``build()`` from code.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libprism_cuda.so")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    srcs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h", "Makefile"))]
    srcs.append(os.path.join(HERE, "..", "include", "prism_cuda.h"))
    return any(os.path.getmtime(s) > t for s in srcs)


def build(force: bool = False, verbose: bool = False) -> str:
    if force or _stale():
        nvcc = os.environ.get("NVCC") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc")
        cmd = ["make", "-C", CSRC, "-j8", f"NVCC={nvcc}"]
        if force:
            subprocess.check_call(["make", "-C", CSRC, "clean"], stdout=subprocess.DEVNULL)
        subprocess.check_call(cmd, stdout=None if verbose else subprocess.DEVNULL)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True))
