"""Builds the CPU oracle (test infrastructure, not product) into oracle/libfg_oracle.so.

Usage: python oracle/build.py
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "fg_oracle.cpp")
OUT = os.path.join(HERE, "libfg_oracle.so")


def build(force: bool = False) -> str:
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= max(os.path.getmtime(SRC),
                                             os.path.getmtime(os.path.join(HERE, "fg_oracle.h")))):
        return OUT
    cmd = ["g++", "-std=c++17", "-O3", "-fopenmp", "-ffp-contract=off", "-fno-math-errno",
           "-shared", "-fPIC", "-o", OUT, SRC]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
