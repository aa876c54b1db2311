"""Compile oracle/linear_oracle.c into oracle/_build/liboracle.so with gcc.

The reference has no compilable CPU code for the Linear path (its arithmetic is
GLSL behind an absent Vulkan wrapper), so there is no oracle/_ref to build; the
C restatement is the only CPU artefact.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "linear_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "liboracle.so")


def build(force=False):
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    # -march=x86-64-v3 (AVX2+FMA) rather than native: the .so is built in one
    # container and executed on another host.  -ffp-contract=off keeps every
    # multiply and add separately rounded, as the restated shader arithmetic is.
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
           "-o", OUT, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
