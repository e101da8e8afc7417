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
SHIM = os.path.join(HERE, "libade_b200_torch.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def sources():
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))] + [
        os.path.join(os.path.dirname(HERE), "include", "ade_b200.h")]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the kernel library and the torch binding when they are missing or older than any of their sources."""
    if force or not (os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in sources())):
        nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), os.path.join(CSRC, "ade_b200.cu"), "-o", LIB + ".tmp"]
        subprocess.run(cmd, check=True)
        os.replace(LIB + ".tmp", LIB)
    build_shim(force)
    return LIB


def build_shim(force: bool = False) -> str:
    """The thin torch binding (csrc/torch_shim.cpp -> libade_b200_torch.so): host compiler only, linked against the
    kernel library next to it (found at run time through $ORIGIN) and against the installed torch."""
    src = os.path.join(CSRC, "torch_shim.cpp")
    header = os.path.join(os.path.dirname(HERE), "include", "ade_b200.h")
    if not force and os.path.exists(SHIM) and all(os.path.getmtime(SHIM) >= os.path.getmtime(s) for s in (src, header, LIB)):
        return SHIM
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths("cuda")
    libs = ce.library_paths("cuda")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", src, "-o", SHIM + ".tmp",
           *[f"-I{i}" for i in inc], *[f"-L{l}" for l in libs], f"-L{HERE}", "-lade_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu",
           "-ltorch_cuda", "-ltorch", "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{l}" for l in libs]]
    subprocess.run(cmd, check=True)
    os.replace(SHIM + ".tmp", SHIM)
    return SHIM


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
