"""Builds the one piece of the reference's path that compiles from its own sources without its
build system: the CUB radix-sort wrapper delaunay_rasterization/internal/sort_by_keys/sort_by_keys.cu
(a torch C++ extension of 59 lines).  It is compiled FROM the reference checkout, where it lies, into
oracle/_ref/ (ignored by git; nothing of the reference is copied into this repository) for sm_100a.
The bench uses it on the GPU as the reference's own sort, timed beside this library's list build
and as a second, independent pin of the tile-list order.

    python oracle/build_ref.py <path-to-reference-checkout>

Needs torch's headers and nvcc; no GPU is needed to build.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "ref_sort_by_keys"


def build(ref_root, verbose=False):
    src = os.path.join(ref_root, "delaunay_rasterization", "internal", "sort_by_keys", "sort_by_keys.cu")
    if not os.path.exists(src):
        return None
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=[src], build_directory=OUT, verbose=verbose,
         extra_cuda_cflags=["-O3", "-gencode", "arch=compute_100a,code=sm_100a"])
    return os.path.join(OUT, NAME + ".so")


def load_prebuilt():
    """Imports oracle/_ref/ref_sort_by_keys.so if it was built; None otherwise."""
    path = os.path.join(OUT, NAME + ".so")
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against torch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", verbose=True))
