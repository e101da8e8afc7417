"""Build recipe of the C oracle (test infrastructure, not product code).

`python oracle/build.py` compiles oracle/ade_oracle.c into oracle/libade_oracle.so with
gcc.  The flags are fixed on purpose: -ffp-contract=off keeps the multiply and the add of
the per-group rescale separate, as the reference's PyTorch code performs them
(src/quantization.py:315); -mavx2 (not -march=native) keeps the binary runnable on a
different x86-64 host than the one that built it.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ade_oracle.c")
LIB = os.path.join(HERE, "libade_oracle.so")
FLAGS = ["-O3", "-mavx2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-std=c11", "-Wall"]


def build(force: bool = False) -> str:
    """Compile the oracle if the shared object is missing or older than its source."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", *FLAGS, SRC, "-o", LIB + ".tmp"]
    subprocess.run(cmd, check=True, cwd=HERE)
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
