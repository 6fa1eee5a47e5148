"""Build recipe for the CPU oracle (test infrastructure, not product code).

Compiles oracle/rm_oracle.cpp and oracle/quad_oracle.cpp into
oracle/librm_oracle.so with g++.  Floating-point contraction is disabled so
that the fp32 stage-1 arithmetic (tile rectangles, sort depths) is the plain
IEEE sequence the CUDA kernels reproduce bit for bit.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = [os.path.join(HERE, "rm_oracle.cpp"), os.path.join(HERE, "quad_oracle.cpp")]
TARGET = os.path.join(HERE, "librm_oracle.so")


def needs_build():
    if not os.path.exists(TARGET):
        return True
    t = os.path.getmtime(TARGET)
    return any(os.path.getmtime(s) > t for s in SOURCES)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return TARGET
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-Wall", "-Wno-unused-variable", "-o", TARGET] + SOURCES
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return TARGET


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
