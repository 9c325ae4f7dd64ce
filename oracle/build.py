"""Compile the CPU oracle (oracle/hc_oracle.c) into oracle/_build/libhc_oracle.so.

Test infrastructure: the shipped library never loads what this builds.
The Honeycrisp reference itself is Swift on top of Apple's Accelerate and cannot be
compiled on Linux, so there is no `oracle/_ref` build of the reference's own sources.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libhc_oracle.so")
SRC = os.path.join(HERE, "hc_oracle.c")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
           "-o", LIB, SRC]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
