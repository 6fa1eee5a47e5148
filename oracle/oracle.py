"""ctypes front-end of the CPU oracle (test infrastructure only).

Only tests/, the smoke test and the bench's CPU-baseline legs may import this
module; the product path never does.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_LIB = None


class OrCamera(C.Structure):
    _fields_ = [("world_view", C.c_float * 16), ("K", C.c_float * 9), ("cam_pos", C.c_float * 3),
                ("distortion", C.c_float * 4), ("image_height", C.c_int), ("image_width", C.c_int),
                ("camera_type", C.c_int), ("fovy", C.c_float), ("fovx", C.c_float), ("min_t", C.c_float),
                ("tile_height", C.c_int), ("tile_width", C.c_int), ("grid_height", C.c_int),
                ("grid_width", C.c_int)]


def lib():
    global _LIB
    if _LIB is None:
        path = _build.build()
        _LIB = C.CDLL(path)
        _LIB.or_count_keys.restype = C.c_int64
        _LIB.or_compute_integral.restype = C.c_float
        _LIB.or_compute_integral.argtypes = [C.c_float, C.c_float, C.c_float]
    return _LIB


def _np(t):
    """Accept numpy arrays or CPU torch tensors."""
    if hasattr(t, "detach"):
        t = t.detach().cpu().numpy()
    return np.asarray(t)


def make_camera(tcam):
    """tcam: dict with the reference's keys (data/camera.py:72-91 + utils/train_util.py:30-37)."""
    c = OrCamera()
    c.world_view[:] = _np(tcam["world_view_transform"]).astype(np.float32).reshape(-1).tolist()
    c.K[:] = _np(tcam["K"]).astype(np.float32).reshape(-1).tolist()
    c.cam_pos[:] = _np(tcam["cam_pos"]).astype(np.float32).reshape(-1).tolist()
    c.distortion[:] = _np(tcam["distortion_params"]).astype(np.float32).reshape(-1).tolist()
    c.image_height = int(tcam["image_height"])
    c.image_width = int(tcam["image_width"])
    c.camera_type = int(tcam["camera_type"])
    c.fovy = float(tcam["fovy"])
    c.fovx = float(tcam["fovx"])
    c.min_t = float(tcam["min_t"])
    c.tile_height = int(tcam["tile_height"])
    c.tile_width = int(tcam["tile_width"])
    c.grid_height = int(tcam["grid_height"])
    c.grid_width = int(tcam["grid_width"])
    return c


def _p(a, ty=None):
    return a.ctypes.data_as(C.c_void_p)


def project(indices, vertices, tcam, nthreads=0):
    """Stage 1. Returns dict(tiles_touched, rect, vs_tetra, circumcenter, nan_seen)."""
    indices = np.ascontiguousarray(_np(indices), dtype=np.int32)
    vertices = np.ascontiguousarray(_np(vertices), dtype=np.float32)
    T = indices.shape[0]
    cam = make_camera(tcam)
    tt = np.zeros(T, np.int32)
    rect = np.zeros((T, 4), np.int32)
    vs = np.zeros((T, 3), np.float32)
    cc = np.zeros((T, 3), np.float32)
    nan_seen = lib().or_project(_p(indices), C.c_int64(T), _p(vertices), C.c_int64(vertices.shape[0]),
                                C.byref(cam), _p(tt), _p(rect), _p(vs), _p(cc), C.c_int(nthreads))
    return dict(tiles_touched=tt, rect=rect, vs_tetra=vs, circumcenter=cc, nan_seen=bool(nan_seen))


def build_lists(tiles_touched, rect, vs_tetra, grid_h, grid_w, want_keys=False):
    """Stages 2-4. Returns (sorted_tetra_idx[N], tile_ranges[G,2][, sorted keys])."""
    tt = np.ascontiguousarray(_np(tiles_touched), dtype=np.int32)
    rect = np.ascontiguousarray(_np(rect), dtype=np.int32)
    vs = np.ascontiguousarray(_np(vs_tetra), dtype=np.float32)
    T = tt.shape[0]
    N = int(lib().or_count_keys(_p(tt), C.c_int64(T)))
    idx = np.zeros(N, np.int32)
    ranges = np.zeros((grid_h * grid_w, 2), np.int32)
    keys = np.zeros(N, np.int64) if want_keys else None
    rc = lib().or_build_lists(_p(tt), _p(rect), _p(vs), C.c_int64(T), C.c_int(grid_h), C.c_int(grid_w),
                              C.c_int64(N), _p(idx), _p(ranges), _p(keys) if want_keys else None)
    assert rc == 0
    return (idx, ranges, keys) if want_keys else (idx, ranges)


def restrict_to_tile_rows(tiles_touched, rect, row0, row1):
    """Clamp every tet rectangle to tile rows [row0, row1): the lists built from the
    result are the single-frame lists of those rows."""
    rect = np.array(_np(rect), dtype=np.int32, copy=True)
    rect[:, 1] = np.maximum(rect[:, 1], row0)
    rect[:, 3] = np.minimum(rect[:, 3], row1)
    h = np.maximum(rect[:, 3] - rect[:, 1], 0)
    tt = ((rect[:, 2] - rect[:, 0]) * h).astype(np.int32)
    tt[np.asarray(_np(tiles_touched)) == 0] = 0
    rect[tt == 0] = 0
    return tt, rect


def _fb_args(dtype, sorted_idx, tile_ranges, indices, vertices, cell_values, jitter):
    return (np.ascontiguousarray(_np(sorted_idx), dtype=np.int32),
            np.ascontiguousarray(_np(tile_ranges), dtype=np.int32),
            np.ascontiguousarray(_np(indices), dtype=np.int32),
            np.ascontiguousarray(_np(vertices), dtype=dtype),
            np.ascontiguousarray(_np(cell_values), dtype=dtype),
            np.ascontiguousarray(_np(jitter), dtype=dtype))


def forward(sorted_idx, tile_ranges, indices, vertices, cell_values, tcam, jitter, rows=None, nthreads=0,
            dtype=np.float32):
    """Stage 5. Returns (output_img[H,W,4], distortion_img[H,W,5], n_contributors[H,W])."""
    sorted_idx, tile_ranges, indices, vertices, cell_values, jitter = _fb_args(
        dtype, sorted_idx, tile_ranges, indices, vertices, cell_values, jitter)
    cam = make_camera(tcam)
    H, W = cam.image_height, cam.image_width
    out = np.zeros((H, W, 4), dtype)
    dist = np.zeros((H, W, 5), dtype)
    nc = np.zeros((H, W), np.int32)
    r0, r1 = rows if rows is not None else (0, H)
    fn = lib().or_forward if dtype == np.float32 else lib().or_forward_f64
    rc = fn(_p(sorted_idx), _p(tile_ranges), _p(indices), _p(vertices), _p(cell_values), C.byref(cam), _p(jitter),
            _p(out), _p(dist), _p(nc), C.c_int(r0), C.c_int(r1), C.c_int(nthreads))
    assert rc == 0
    return out, dist, nc


def forward_constant_color(sorted_idx, tile_ranges, indices, vertices, rgbs, tcam, pre_multi=100.0, ladder_p=-0.1,
                           nthreads=0):
    """Constant-colour debug renderer, forward. rgbs[T,4] = (r, g, b, density).
    Returns (output_img[H,W,4] = (r,g,b,transmittance), distortion_img[H,W,4], n_contributors[H,W])."""
    sorted_idx = np.ascontiguousarray(_np(sorted_idx), np.int32)
    tile_ranges = np.ascontiguousarray(_np(tile_ranges), np.int32)
    indices = np.ascontiguousarray(_np(indices), np.int32)
    vertices = np.ascontiguousarray(_np(vertices), np.float32)
    rgbs = np.ascontiguousarray(_np(rgbs), np.float32)
    cam = make_camera(tcam)
    H, W = cam.image_height, cam.image_width
    out = np.zeros((H, W, 4), np.float32)
    dist = np.zeros((H, W, 4), np.float32)
    nc = np.zeros((H, W), np.int32)
    rc = lib().or_forward_constant_color(_p(sorted_idx), _p(tile_ranges), _p(indices), _p(vertices), _p(rgbs),
                                         C.byref(cam), C.c_float(pre_multi), C.c_float(ladder_p), _p(out), _p(dist),
                                         _p(nc), C.c_int(nthreads))
    assert rc == 0
    return out, dist, nc


def _cc_args(dtype, sorted_idx, tile_ranges, indices, vertices, rgbs):
    return (np.ascontiguousarray(_np(sorted_idx), np.int32), np.ascontiguousarray(_np(tile_ranges), np.int32),
            np.ascontiguousarray(_np(indices), np.int32), np.ascontiguousarray(_np(vertices), dtype),
            np.ascontiguousarray(_np(rgbs), dtype))


def forward_constant_color_f64(sorted_idx, tile_ranges, indices, vertices, rgbs, tcam, pre_multi=100.0, ladder_p=-0.1):
    """The same forward pass in float64 (for finite-difference checks of the backward pass)."""
    sorted_idx, tile_ranges, indices, vertices, rgbs = _cc_args(np.float64, sorted_idx, tile_ranges, indices, vertices,
                                                                rgbs)
    cam = make_camera(tcam)
    H, W = cam.image_height, cam.image_width
    out, dist, nc = np.zeros((H, W, 4)), np.zeros((H, W, 4)), np.zeros((H, W), np.int32)
    rc = lib().or_forward_constant_color_f64(_p(sorted_idx), _p(tile_ranges), _p(indices), _p(vertices), _p(rgbs),
                                             C.byref(cam), C.c_double(pre_multi), C.c_double(ladder_p), _p(out),
                                             _p(dist), _p(nc), C.c_int(0))
    assert rc == 0
    return out, dist, nc


def backward_constant_color(sorted_idx, tile_ranges, indices, vertices, rgbs, tcam, out_img, dist_img, n_contrib,
                            g_img, g_dist, pre_multi=100.0, ladder_p=-0.1, dtype=np.float32, nthreads=0,
                            min_alpha=1.0 / 255.0):
    """Backward of the constant-colour renderer as the reference runs it (slang/alphablend_shader.slang:186-277).
    Returns (vertices_grad[V,3], rgbs_grad[T,4])."""
    sorted_idx, tile_ranges, indices, vertices, rgbs = _cc_args(dtype, sorted_idx, tile_ranges, indices, vertices, rgbs)
    cam = make_camera(tcam)
    arrs = [np.ascontiguousarray(_np(a), dtype) for a in (out_img, dist_img, g_img, g_dist)]
    nc = np.ascontiguousarray(_np(n_contrib), np.int32)
    vg, rg = np.zeros_like(vertices), np.zeros_like(rgbs)
    if dtype == np.float32:
        fn, ft = lib().or_backward_constant_color, C.c_float
    else:
        fn, ft = lib().or_backward_constant_color_f64, C.c_double
    rc = fn(_p(sorted_idx), _p(tile_ranges), _p(indices), _p(vertices), _p(rgbs), C.byref(cam), ft(pre_multi),
            ft(ladder_p), _p(arrs[0]), _p(arrs[1]), _p(nc), _p(arrs[2]), _p(arrs[3]), _p(vg), _p(rg), ft(min_alpha),
            C.c_int(nthreads))
    assert rc == 0
    return vg, rg


def backward(sorted_idx, tile_ranges, indices, vertices, cell_values, tcam, jitter, out_img, dist_img, n_contrib,
             g_img, g_dist, rows=None, nthreads=0, dtype=np.float32):
    """Stage 6. Returns (vertices_grad[V,3], cell_values_grad[T,7])."""
    sorted_idx, tile_ranges, indices, vertices, cell_values, jitter = _fb_args(
        dtype, sorted_idx, tile_ranges, indices, vertices, cell_values, jitter)
    cam = make_camera(tcam)
    H = cam.image_height
    out_img = np.ascontiguousarray(_np(out_img), dtype=dtype)
    dist_img = np.ascontiguousarray(_np(dist_img), dtype=dtype)
    n_contrib = np.ascontiguousarray(_np(n_contrib), dtype=np.int32)
    g_img = np.ascontiguousarray(_np(g_img), dtype=dtype)
    g_dist = np.ascontiguousarray(_np(g_dist), dtype=dtype)
    vg = np.zeros_like(vertices)
    cg = np.zeros_like(cell_values)
    r0, r1 = rows if rows is not None else (0, H)
    fn = lib().or_backward if dtype == np.float32 else lib().or_backward_f64
    rc = fn(_p(sorted_idx), _p(tile_ranges), _p(indices), _p(vertices), _p(cell_values), C.byref(cam), _p(jitter),
            _p(out_img), _p(dist_img), _p(n_contrib), _p(g_img), _p(g_dist), _p(vg), _p(cg), C.c_int(r0),
            C.c_int(r1), C.c_int(nthreads))
    assert rc == 0
    return vg, cg


def sensitive_pixels(sorted_idx, tile_ranges, indices, vertices, cell_values, tcam, jitter, tol=1e-4, nthreads=0,
                     flags=False):
    """Boolean [H,W] mask of pixels decided by rounding in the reference algorithm itself.  With flags=True
    the uint8 flags instead: bit 0 = a grazing ray/tet contact, bit 1 = a log-transmittance within tol (relative)
    of the termination cut-off."""
    sorted_idx, tile_ranges, indices, vertices, cell_values, jitter = _fb_args(
        np.float32, sorted_idx, tile_ranges, indices, vertices, cell_values, jitter)
    cam = make_camera(tcam)
    mask = np.zeros((cam.image_height, cam.image_width), np.uint8)
    lib().or_sensitive_pixels(_p(sorted_idx), _p(tile_ranges), _p(indices), _p(vertices), _p(cell_values),
                              C.byref(cam), _p(jitter), _p(mask), C.c_float(tol), C.c_int(nthreads))
    return mask if flags else mask.astype(bool)


def tet_err(sorted_idx, tile_ranges, indices, vertices, cell_values, tcam, pixel_err, ssim_err, nthreads=0):
    """Densification statistics. Returns (tet_err[T,16] f32, tet_count[T,2] i32)."""
    jit = np.zeros((1, 1, 2), np.float32)
    sorted_idx, tile_ranges, indices, vertices, cell_values, _ = _fb_args(
        np.float32, sorted_idx, tile_ranges, indices, vertices, cell_values, jit)
    cam = make_camera(tcam)
    pe = np.ascontiguousarray(_np(pixel_err), dtype=np.float32)
    se = np.ascontiguousarray(_np(ssim_err), dtype=np.float32)
    T = indices.shape[0]
    err = np.zeros((T, 16), np.float32)
    cnt = np.zeros((T, 2), np.int32)
    lib().or_tet_err(_p(sorted_idx), _p(tile_ranges), _p(indices), _p(vertices), _p(cell_values), C.byref(cam),
                     _p(pe), _p(se), C.c_int64(T), _p(err), _p(cnt), C.c_int(nthreads))
    return err, cnt


def vertex_backward(indices, vertices, tcam, tiles_touched, g_vs, g_cc):
    """Reverse of stage 1 wrt vertices. Returns vertices_grad[V,3]."""
    indices = np.ascontiguousarray(_np(indices), dtype=np.int32)
    vertices = np.ascontiguousarray(_np(vertices), dtype=np.float32)
    tt = np.ascontiguousarray(_np(tiles_touched), dtype=np.int32)
    g_vs = np.ascontiguousarray(_np(g_vs), dtype=np.float32)
    g_cc = np.ascontiguousarray(_np(g_cc), dtype=np.float32)
    cam = make_camera(tcam)
    vg = np.zeros_like(vertices)
    lib().or_vertex_backward(_p(indices), C.c_int64(indices.shape[0]), _p(vertices), C.byref(cam), _p(tt), _p(g_vs),
                             _p(g_cc), _p(vg))
    return vg


def power_f64(verts4x3, P):
    v = np.ascontiguousarray(verts4x3, dtype=np.float64)
    P = np.ascontiguousarray(P, dtype=np.float64)
    power = C.c_double()
    center = np.zeros(3, np.float64)
    lib().or_power_f64(_p(v), _p(P), C.byref(power), _p(center))
    return power.value, center


def compute_integral(c0, c1, ddt):
    return float(lib().or_compute_integral(C.c_float(c0), C.c_float(c1), C.c_float(ddt)))


def num_threads():
    return int(lib().or_num_threads())


def render(indices, vertices, cell_values, tcam, jitter=None, nthreads=0):
    """Whole forward path on the CPU: stages 1-5."""
    H, W = int(tcam["image_height"]), int(tcam["image_width"])
    if jitter is None:
        jitter = np.full((H, W, 2), 0.5, np.float32)
    pr = project(indices, vertices, tcam, nthreads)
    idx, ranges = build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], int(tcam["grid_height"]),
                              int(tcam["grid_width"]))
    out, dist, nc = forward(idx, ranges, indices, vertices, cell_values, tcam, jitter, nthreads=nthreads)
    return dict(project=pr, sorted_idx=idx, tile_ranges=ranges, output_img=out, distortion_img=dist,
                n_contributors=nc)


def quad_render(vertices, indices, vertex_color, tet_density, height, width, viewmat, fx, fy, tmin, n_samples,
                pixels=None, grd_mode=0, want_grad=False, nthreads=0):
    """Quadrature renderer (jaxutil/tetra_quad.py:275-311). Returns [npix,5] (+ grads)."""
    vertices = np.ascontiguousarray(_np(vertices), dtype=np.float32)
    indices = np.ascontiguousarray(_np(indices), dtype=np.int32)
    vc = np.ascontiguousarray(_np(vertex_color), dtype=np.float32).reshape(-1, 6)
    td = np.ascontiguousarray(_np(tet_density), dtype=np.float32).reshape(-1)
    vm = np.ascontiguousarray(_np(viewmat), dtype=np.float32)
    p0, p1 = pixels if pixels is not None else (0, height * width)
    out = np.zeros((p1 - p0, 5), np.float32)
    T = indices.shape[0]
    gd = np.zeros(T, np.float64) if want_grad else None
    gc = np.zeros((T, 6), np.float64) if want_grad else None
    rc = lib().quad_render(_p(vertices), C.c_int64(vertices.shape[0]), _p(indices), C.c_int64(T), _p(vc), _p(td),
                           C.c_int(height), C.c_int(width), _p(vm), C.c_float(fx), C.c_float(fy), C.c_float(tmin),
                           C.c_int(n_samples), C.c_int64(p0), C.c_int64(p1), C.c_int(grd_mode), _p(out),
                           _p(gd) if want_grad else None, _p(gc) if want_grad else None, C.c_int(nthreads))
    assert rc == 0
    return (out, gd, gc) if want_grad else out
