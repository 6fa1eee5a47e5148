"""Seeded synthetic scenes and cameras standing in for the reference's trained
checkpoints and datasets (which need a network to fetch).

The five generators follow the benchmark configurations: uniform cube
(CPU-runnable), Gaussian mixture, and the unbounded-scene mixture of a clustered
foreground plus spherical shells, each tetrahedralised with scipy's Delaunay.
Everything is NumPy on the host; callers move the arrays to the GPU.

Cameras follow the reference's tcam dictionary (data/camera.py:72-91 plus the
tile fields added in utils/train_util.py:30-37): world_view_transform is the
row-major world->camera matrix, K the 3x3 pinhole intrinsics with the principal
point at the image centre, cam_pos the camera centre.
"""
import math

import numpy as np


def orient_positive(points, tets):
    """Swap two indices of negatively oriented tets (models/ingp_color.py:526-531)."""
    v = points[tets]
    vol = np.einsum("ij,ij->i", np.cross(v[:, 1] - v[:, 0], v[:, 2] - v[:, 0]), v[:, 3] - v[:, 0])
    tets = tets.copy()
    neg = vol < 0
    tets[neg] = tets[neg][:, [1, 0, 2, 3]]
    return tets


def delaunay(points):
    from scipy.spatial import Delaunay
    tri = Delaunay(points.astype(np.float64))
    return orient_positive(points.astype(np.float64), tri.simplices.astype(np.int32)).astype(np.int32)


def _features(rng, T, mu, sigma, zero_frac=0.0):
    density = rng.lognormal(mu, sigma, T).astype(np.float32)
    if zero_frac > 0:
        density[rng.random(T) < zero_frac] = 0.0
    base = rng.uniform(0, 1, (T, 3)).astype(np.float32)
    grd = rng.normal(0, 0.5, (T, 3)).astype(np.float32)
    return np.concatenate([density[:, None], base, grd], axis=1).astype(np.float32)


def points_uniform(n, seed=0):
    return np.random.default_rng(seed).uniform(-1, 1, (n, 3)).astype(np.float32)


def points_gaussians(n, n_clusters=8, sigma=0.15, seed=1):
    rng = np.random.default_rng(seed)
    centers = rng.uniform(-1, 1, (n_clusters, 3))
    pts = centers[rng.integers(0, n_clusters, n)] + rng.normal(0, sigma, (n, 3))
    return pts.astype(np.float32)


def points_unbounded(n, n_clusters=16, sigma=0.1, seed=2):
    """70 % clustered foreground in the unit ball, 30 % on shells of radius 2..10."""
    rng = np.random.default_rng(seed)
    nf = int(0.7 * n)
    c = rng.normal(size=(n_clusters, 3))
    c = c / np.linalg.norm(c, axis=1, keepdims=True) * rng.uniform(0, 0.7, (n_clusters, 1))
    fg = c[rng.integers(0, n_clusters, nf)] + rng.normal(0, sigma, (nf, 3))
    nb = n - nf
    d = rng.normal(size=(nb, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    bg = d * rng.uniform(2, 10, (nb, 1))
    return np.concatenate([fg, bg]).astype(np.float32)


def make_scene(config, n_points=None):
    """Returns dict(vertices[V,3] f32, indices[T,4] i32, cell_values[T,7] f32, name)."""
    if config == 1:
        pts = points_uniform(n_points or 2000, seed=0)
        mu, sg, zf = 0.0, 1.0, 0.0
    elif config == 2:
        pts = points_gaussians(n_points or 100_000, seed=1)
        mu, sg, zf = -1.0, 1.5, 0.0
    elif config in (3, 4, 5):
        default = {3: 1_000_000, 4: 3_000_000, 5: 5_000_000}[config]
        pts = points_unbounded(n_points or default, seed=2)
        mu, sg, zf = -0.5, 2.0, 0.4
    else:
        raise ValueError(f"unknown config {config}")
    tets = delaunay(pts)
    rng = np.random.default_rng(100 + config)
    cell = _features(rng, tets.shape[0], mu, sg, zf)
    return dict(vertices=pts, indices=tets, cell_values=cell, name=f"config{config}")


def look_at(eye, target=(0.0, 0.0, 0.0), up=(0.0, 1.0, 0.0)):
    """World->camera 4x4 (camera looks along +z), tests/multi_tet_test.py:27-43."""
    eye = np.asarray(eye, np.float64)
    fwd = np.asarray(target, np.float64) - eye
    fwd /= np.linalg.norm(fwd)
    right = np.cross(fwd, np.asarray(up, np.float64))
    if np.linalg.norm(right) < 1e-6:
        right = np.cross(fwd, np.array([1.0, 0, 0]))
    right /= np.linalg.norm(right)
    upv = np.cross(right, fwd)
    c2w = np.eye(4)
    c2w[:3, 0], c2w[:3, 1], c2w[:3, 2], c2w[:3, 3] = right, upv, fwd, eye
    return np.linalg.inv(c2w)


def make_tcam(viewmat, height, width, fov_deg, tile=4, min_t=0.1, camera_type=0, distortion=None):
    """tcam dictionary with NumPy values (the caller converts the arrays to device tensors).
    `tile` is the tile edge in pixels, or (tile_height, tile_width)."""
    tile_h, tile_w = (tile, tile) if isinstance(tile, int) else (int(tile[0]), int(tile[1]))
    fovy = math.radians(fov_deg)
    fy = height / (2 * math.tan(fovy / 2))
    fx = fy
    fovx = 2 * math.atan(width / (2 * fx))
    vm = np.asarray(viewmat, np.float64)
    cam_pos = np.linalg.inv(vm)[:3, 3]
    return dict(
        world_view_transform=vm.astype(np.float32),
        cam_pos=cam_pos.astype(np.float32),
        K=np.array([[fx, 0, width / 2], [0, fy, height / 2], [0, 0, 1]], np.float32),
        image_height=int(height), image_width=int(width), fovy=float(fovy), fovx=float(fovx),
        distortion_params=np.zeros(4, np.float32) if distortion is None else np.asarray(distortion, np.float32),
        camera_type=int(camera_type),
        tile_height=tile_h, tile_width=tile_w,
        grid_height=(height + tile_h - 1) // tile_h, grid_width=(width + tile_w - 1) // tile_w,
        min_t=float(min_t),
    )


def ring_camera(k, n_views, height, width, fov_deg, radius=3.0, **kw):
    ang = 2 * math.pi * k / max(n_views, 1)
    eye = (radius * math.cos(ang), 0.0, radius * math.sin(ang))
    return make_tcam(look_at(eye), height, width, fov_deg, **kw)


CONFIG_CAMERAS = {
    1: dict(height=128, width=128, fov_deg=60.0),
    2: dict(height=800, width=800, fov_deg=50.0),
    3: dict(height=1080, width=1920, fov_deg=60.0),
    4: dict(height=1080, width=1920, fov_deg=60.0),
    5: dict(height=2160, width=3840, fov_deg=90.0),
}


def config_camera(config, view=0, n_views=8, **kw):
    c = dict(CONFIG_CAMERAS[config])
    c.update(kw)
    if config == 1:
        return make_tcam(look_at((0.0, 0.0, 3.0)), **c)
    return ring_camera(view, n_views, **c)
