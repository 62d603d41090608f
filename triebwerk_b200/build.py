"""Builds csrc/libtriebwerk_b200.so in-tree with nvcc for sm_100a (``python -m triebwerk_b200.build``)."""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB = os.path.join(CSRC, "libtriebwerk_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-shared", "-Xcompiler",
         "-fPIC"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))) + [
        os.path.join(os.path.dirname(_HERE), "include", "triebwerk_b200.h")]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than any source.  Returns its path."""
    if not force and os.path.exists(LIB):
        newest = max(os.path.getmtime(s) for s in sources())
        if os.path.getmtime(LIB) >= newest:
            return LIB
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB, os.path.join(CSRC, "tq_capi.cu")]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
