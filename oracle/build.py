"""Compile the CPU oracle (test infrastructure) into oracle/_build/liboracle.so.

Contraction is disabled on purpose: the reference's scalar Go code never fuses
a*b+c on amd64, and the AVX2 paths are restated with explicit fmaf().
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "oracle.cpp")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "liboracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= os.path.getmtime(SRC)):
        return LIB
    cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fno-fast-math",
           "-fvisibility=hidden", "-shared", "-fPIC", "-pthread", SRC, "-o", LIB]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
