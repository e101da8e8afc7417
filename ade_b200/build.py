"""Build recipe of libade_b200.so (the CUDA kernels behind the C ABI of include/ade_b200.h).

`python -m ade_b200.build` compiles ade_b200/csrc/ade_b200.cu for sm_100a with nvcc and puts
the shared object next to this file, where ade_b200._lib loads it.  nvcc cross-compiles, so
the build needs no GPU.  The explicit -gencode form is required: tcgen05 instructions only
exist for the architecture-specific target sm_100a.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libade_b200.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def sources():
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))] + [
        os.path.join(os.path.dirname(HERE), "include", "ade_b200.h")]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library when it is missing or older than any of its sources."""
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in sources()):
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), os.path.join(CSRC, "ade_b200.cu"), "-o", LIB + ".tmp"]
    subprocess.run(cmd, check=True)
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
