"""Build the CPU oracle (test infrastructure, never part of the product library).

Two shared objects from the one source file:
  libholo_oracle.so       parity build  (-O2 -ffp-contract=off -fno-fast-math)
  libholo_oracle_fast.so  timing build  (-O3 -march=x86-64-v3 -fopenmp), CPU-baseline legs only

Run: python oracle/build.py
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "hologram_oracle.c")
PARITY = os.path.join(HERE, "libholo_oracle.so")
FAST = os.path.join(HERE, "libholo_oracle_fast.so")


def _stale(out):
    return not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(SRC)


def build(force=False):
    common = ["gcc", "-std=c11", "-shared", "-fPIC", "-fno-fast-math", "-Wall", "-Wno-unknown-pragmas"]
    if force or _stale(PARITY):
        subprocess.check_call(common + ["-O2", "-ffp-contract=off", "-fopenmp", SRC, "-o", PARITY, "-lm"])
    if force or _stale(FAST):
        subprocess.check_call(common + ["-O3", "-march=x86-64-v3", "-fopenmp", SRC, "-o", FAST, "-lm"])
    return PARITY, FAST


if __name__ == "__main__":
    print(*build(force="--force" in sys.argv), sep="\n")
