"""Ahead-of-time build of librm_b200.so for sm_100a with nvcc.

The projection unit is compiled with -fmad=false (its fp32/fp64 arithmetic
decides the tile lists and must be the plain IEEE sequence); the other units
may contract freely.  The library is written next to the package so that it
travels with the source tree.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
TARGET = os.path.join(PKG, "librm_b200.so")
UNITS = [("rm_project.cu", ["-fmad=false"]), ("rm_binning.cu", []), ("rm_raster.cu", []), ("rm_activate.cu", []),
         ("rm_multimem.cu", []), ("rm_api.cu", [])]
HEADERS = [os.path.join(HERE, "rm_common.cuh"), os.path.join(INCLUDE, "rm_b200.h")]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _target(variant):
    return TARGET if variant is None else os.path.join(PKG, f"librm_b200_{variant}.so")


def needs_build(variant=None):
    target = _target(variant)
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    srcs = [os.path.join(HERE, u) for u, _ in UNITS] + HEADERS + [os.path.abspath(__file__)]
    return any(os.path.getmtime(s) > t for s in srcs)


def build(force=False, verbose=False, ptxas_info=False, variant=None):
    """variant=None: the library.  variant="check": the bounds-checked build (-DRM_BOUNDS_CHECK), written to
    librm_b200_check.so and loaded by the tests through RM_B200_LIBRARY."""
    assert variant in (None, "check")
    target = _target(variant)
    if not force and not needs_build(variant):
        return target
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build" if variant is None else f"build_{variant}")
    os.makedirs(objdir, exist_ok=True)
    defines = ["-DRM_BOUNDS_CHECK"] if variant == "check" else []
    objs = []
    for unit, extra in UNITS:
        obj = os.path.join(objdir, unit.replace(".cu", ".o"))
        cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", *ARCH, "-I", INCLUDE, "-I", HERE, "-Xcompiler", "-fPIC",
               *defines, *extra, "-c", os.path.join(HERE, unit), "-o", obj]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        objs.append(obj)
    # link beside the target and rename: a reader never sees a half-written library
    tmp = target + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", *ARCH, "-o", tmp, *objs]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    os.replace(tmp, target)
    return target


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv,
          variant="check" if "--check" in sys.argv else None)
