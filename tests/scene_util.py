"""Seeded small scenes shared by the CPU and GPU tests."""
import numpy as np

from radiance_meshes_b200 import scenes


def small_scene(n_points=300, seed=0, mu=0.0, sigma=1.0, zero_frac=0.2, scale=1.0):
    pts = (scenes.points_uniform(n_points, seed=seed) * scale).astype(np.float32)
    tets = scenes.delaunay(pts)
    rng = np.random.default_rng(seed + 1000)
    cell = scenes._features(rng, tets.shape[0], mu, sigma, zero_frac)
    return pts, tets, cell


def camera(eye=(0.3, 0.2, 2.5), H=64, W=64, fov=60.0, tile=4, min_t=0.1, **kw):
    return scenes.make_tcam(scenes.look_at(eye), H, W, fov, tile=tile, min_t=min_t, **kw)


def jitter(H, W, seed=0):
    return np.random.default_rng(seed).uniform(0.05, 0.95, (H, W, 2)).astype(np.float32)
