"""Regenerates tests/golden/small_scene.npz: a seeded 80-point scene with the CPU
oracle's outputs for every stage.  The reference stores no golden vectors for
this path and cannot be executed without the Slang compiler and JAX, so these
vectors pin the oracle against regressions and give the GPU tests a fixture that
does not depend on rebuilding the oracle.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle as O  # noqa: E402
import scene_util  # noqa: E402


def main():
    pts, tets, cell = scene_util.small_scene(80, seed=11)
    H = W = 32
    tcam = scene_util.camera(eye=(0.4, -0.3, 2.2), H=H, W=W, tile=4)
    jit = scene_util.jitter(H, W, seed=3)
    r = O.render(tets, pts, cell, tcam, jit)
    rng = np.random.default_rng(5)
    g_img = rng.normal(size=(H, W, 4)).astype(np.float32)
    g_dist = (0.05 * rng.normal(size=(H, W, 5))).astype(np.float32)
    vg, cg = O.backward(r["sorted_idx"], r["tile_ranges"], tets, pts, cell, tcam, jit, r["output_img"],
                        r["distortion_img"], r["n_contributors"], g_img, g_dist)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "small_scene.npz")
    np.savez_compressed(
        out, vertices=pts, indices=tets, cell_values=cell, jitter=jit, eye=np.array([0.4, -0.3, 2.2]),
        H=H, W=W, tile=4, fov=60.0, min_t=0.1,
        tiles_touched=r["project"]["tiles_touched"], rect=r["project"]["rect"], vs_tetra=r["project"]["vs_tetra"],
        circumcenter=r["project"]["circumcenter"], sorted_idx=r["sorted_idx"], tile_ranges=r["tile_ranges"],
        output_img=r["output_img"], distortion_img=r["distortion_img"], n_contributors=r["n_contributors"],
        g_img=g_img, g_dist=g_dist, vertices_grad=vg, cell_grad=cg)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
