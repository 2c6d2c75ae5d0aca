"""Compile the CPU oracle (test infrastructure) into oracle/liboracle.so.

Flags matter for the bits: -ffp-contract=off because the reference's JIT never
fuses a*b+c, and no -ffast-math so summation order is exactly as written.
-mavx2 (not -march=native) because the library is built on one machine and
carried to another.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "cpu_matmul.c")
OUT = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O2", "-mavx2", "-ffp-contract=off", "-fPIC", "-shared", "-pthread",
           "-o", OUT, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
