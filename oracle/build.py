"""Build recipe for the CPU oracle (test infrastructure, never shipped).

    python oracle/build.py

compiles oracle/forge_oracle.c into oracle/libforge_oracle.so with gcc.  The
flags are part of the oracle's definition: -ffp-contract=off keeps every fused
multiply-add explicit, and -fno-fast-math keeps IEEE rounding.  -mavx2 -mfma let
the compiler use the hardware fused multiply-add for fmaf() (exactly rounded,
so bit-identical to the library routine) and vectorise the row loops; they do
not change any result, only how long the CPU baseline takes.

The reference has no CPU implementation of its CUDA kernels and its Python half
needs no compilation, so there is nothing to build into oracle/_ref.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "forge_oracle.c")
OUT = os.path.join(HERE, "libforge_oracle.so")


def build(force: bool = False) -> str:
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)):
        return OUT
    cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-fPIC",
           "-shared", "-o", OUT, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
