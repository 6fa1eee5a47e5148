"""CPU tests of the oracle itself: known answers, finite differences, the
independent quadrature restatement, structural properties of the tile lists and
the committed golden fixture."""
import os

import numpy as np
import pytest

import scene_util
from radiance_meshes_b200 import scenes

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "small_scene.npz")


def test_integral_known_answer(oracle):
    # notebooks/integral.ipynb cell 0: compute_integral(1, 1, dt=2, d=1) == 1 - exp(-2)
    assert abs(oracle.compute_integral(1.0, 1.0, 2.0) - (1 - np.exp(-2.0))) < 1e-6
    # the same notebook's closed form for unequal end colours
    for c0, c1, tau in [(0.2, 0.9, 0.5), (1.0, 0.0, 3.0), (0.3, 0.7, 1e-3), (0.5, 0.25, 20.0)]:
        a = np.exp(-tau)
        ref = ((-tau * a + 1 - a) * c0 + ((tau - 1) + a) * c1) / tau
        assert abs(oracle.compute_integral(c0, c1, tau) - ref) < 2e-5 * max(1.0, abs(ref)) + 1e-6


def test_sortable_key_order(oracle):
    # keys of a sorted list must be non-decreasing within each tile
    pts, tets, cell = scene_util.small_scene(200, seed=2)
    tcam = scene_util.camera(H=48, W=40, tile=8)
    pr = oracle.project(tets, pts, tcam)
    idx, ranges, keys = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], tcam["grid_height"],
                                           tcam["grid_width"], want_keys=True)
    assert idx.shape[0] == pr["tiles_touched"].sum()
    assert np.all(np.diff(keys.astype(np.uint64)) >= 0)
    depth = pr["vs_tetra"][:, 2]
    covered = 0
    for t, (s, e) in enumerate(ranges):
        if e == s:
            assert (s, e) == (0, 0)
            continue
        seg = idx[s:e]
        d = depth[seg]
        assert np.all(np.diff(d) >= 0)
        # ties broken by tet id
        same = np.diff(d) == 0
        assert np.all(np.diff(seg)[same] > 0)
        ty, tx = divmod(t, tcam["grid_width"])
        r = pr["rect"][seg]
        assert np.all((r[:, 0] <= tx) & (tx < r[:, 2]) & (r[:, 1] <= ty) & (ty < r[:, 3]))
        covered += e - s
    assert covered == idx.shape[0]


def test_backward_matches_finite_differences_f64(oracle):
    rng = np.random.default_rng(5)
    pts, tets, cell = scene_util.small_scene(60, seed=3)
    H = W = 24
    tcam = scene_util.camera(H=H, W=W)
    pr = oracle.project(tets, pts, tcam)
    idx, ranges = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], tcam["grid_height"],
                                     tcam["grid_width"])
    jit = rng.uniform(0.2, 0.8, (H, W, 2))
    wi = rng.normal(size=(H, W, 4))
    wd = rng.normal(size=(H, W, 5)) * 0.1
    v64, c64 = pts.astype(np.float64), cell.astype(np.float64)

    def loss(v, c):
        out, dist, nc = oracle.forward(idx, ranges, tets, v, c, tcam, jit, dtype=np.float64)
        return (out * wi).sum() + (dist * wd).sum(), out, dist, nc

    _, out, dist, nc = loss(v64, c64)
    vg, cg = oracle.backward(idx, ranges, tets, v64, c64, tcam, jit, out, dist, nc, wi, wd, dtype=np.float64)
    eps = 1e-6
    scale = np.abs(vg).max()
    for _ in range(20):
        i, k = rng.integers(0, pts.shape[0]), rng.integers(0, 3)
        vp, vm = v64.copy(), v64.copy()
        vp[i, k] += eps
        vm[i, k] -= eps
        fd = (loss(vp, c64)[0] - loss(vm, c64)[0]) / (2 * eps)
        assert abs(fd - vg[i, k]) < 1e-5 * scale + 1e-6
    scale = np.abs(cg).max()
    for _ in range(30):
        i, k = rng.integers(0, tets.shape[0]), rng.integers(0, 7)
        if k == 0 and cell[i, 0] == 0:
            continue  # kink of max(density, 0): the reference gives no gradient there
        cp, cm = c64.copy(), c64.copy()
        cp[i, k] += eps
        cm[i, k] -= eps
        fd = (loss(v64, cp)[0] - loss(v64, cm)[0]) / (2 * eps)
        assert abs(fd - cg[i, k]) < 1e-5 * scale + 1e-6


def test_vertex_backward_matches_finite_differences(oracle):
    rng = np.random.default_rng(1)
    P = np.array([0.3, -0.2, 2.0])
    for _ in range(5):
        v = rng.normal(size=(4, 3))
        gp, gc = rng.normal(), rng.normal(size=3)
        tcam = scene_util.camera(eye=tuple(P))
        tcam["cam_pos"] = P.astype(np.float32)
        vg = oracle.vertex_backward(np.array([[0, 1, 2, 3]], np.int32), v.astype(np.float32), tcam,
                                    np.array([1], np.int32), np.array([[0, 0, gp]], np.float32),
                                    gc[None].astype(np.float32))
        v32 = v.astype(np.float32).astype(np.float64)
        P32 = P.astype(np.float32).astype(np.float64)
        eps = 1e-6
        for i in range(4):
            for k in range(3):
                a, b = v32.copy(), v32.copy()
                a[i, k] += eps
                b[i, k] -= eps
                pa, ca = oracle.power_f64(a, P32)
                pb, cb = oracle.power_f64(b, P32)
                fd = ((pa - pb) * gp + ((ca - cb) * gc).sum()) / (2 * eps)
                assert abs(fd - vg[i, k]) < 1e-4 * max(1.0, abs(fd))


def test_rasterizer_agrees_with_quadrature(oracle):
    # the reference's own check (tests/multi_tet_test.py:13-18): image and
    # gradients within 1e-1 of the quadrature, error shrinking with sample count
    rng = np.random.default_rng(7)
    pts = rng.uniform(-1, 1, (20, 3)).astype(np.float32)
    tets = scenes.delaunay(pts)
    T = tets.shape[0]
    cell = np.concatenate([np.ones((T, 1)), rng.uniform(0.2, 1, (T, 3)), rng.normal(0, 0.1, (T, 3))], 1).astype(
        np.float32)
    H = W = 16
    tcam = scenes.make_tcam(scenes.look_at((0.5, 0.4, 3.0)), H, W, 50.0, tile=8, min_t=0.01)
    r = oracle.render(tets, pts, cell, tcam)
    img = r["output_img"]
    fx, fy = float(tcam["K"][0, 0]), float(tcam["K"][1, 1])
    errs = []
    for ns in (256, 1024):
        q = oracle.quad_render(pts, tets, cell[:, 1:], cell[:, 0], H, W, tcam["world_view_transform"], fx, fy, 0.01,
                               ns).reshape(H, W, 5)
        errs.append(np.abs(q[..., :3] - img[..., :3]).mean())
        np.testing.assert_allclose(q[..., :3], img[..., :3], atol=1e-1, rtol=1e-1)
        np.testing.assert_allclose(q[..., 3], 1 - np.exp(img[..., 3]), atol=1e-1, rtol=1e-1)
    assert errs[1] < errs[0]
    gi = np.zeros((H, W, 4), np.float32)
    gi[..., :3] = 1
    vg, cg = oracle.backward(r["sorted_idx"], r["tile_ranges"], tets, pts, cell, tcam,
                             np.full((H, W, 2), 0.5, np.float32), r["output_img"], r["distortion_img"],
                             r["n_contributors"], gi, np.zeros((H, W, 5), np.float32))
    q, gd, gc = oracle.quad_render(pts, tets, cell[:, 1:], cell[:, 0], H, W, tcam["world_view_transform"], fx, fy,
                                   0.01, 1024, want_grad=True)
    np.testing.assert_allclose(gd, cg[:, 0], atol=1e-1, rtol=1e-1)
    np.testing.assert_allclose(gc, cg[:, 1:], atol=1e-1, rtol=1e-1)


def test_single_tet_views(oracle):
    # tests/single_tet_test.py: one tet, camera inside it and outside it
    rng = np.random.default_rng(189710234 % 2**32)
    v = ((rng.random((4, 3)) * 2 - 1) * 0.4).astype(np.float32)
    tets = scenes.orient_positive(v.astype(np.float64), np.array([[0, 1, 2, 3]], np.int32)).astype(np.int32)
    cell = np.array([[10.0, 0.25, 0.5, 0.1, -0.15, 0.25, 0.1]], np.float32)
    H = W = 32
    inside = v.mean(0)
    for eye, expect_all in ((tuple(inside), True), ((0.0, 0.0, 3.0), False)):
        target = (0.0, 0.0, 0.0) if not expect_all else tuple(inside + np.array([0, 0, 1.0]))
        tcam = scenes.make_tcam(scenes.look_at(eye, target), H, W, 90.0, tile=16, min_t=0.01)
        r = oracle.render(tets, v, cell, tcam)
        fx = float(tcam["K"][0, 0])
        q = oracle.quad_render(v, tets, cell[:, 1:], cell[:, 0], H, W, tcam["world_view_transform"], fx, fx, 0.01,
                               2000).reshape(H, W, 5)
        np.testing.assert_allclose(q[..., :3], r["output_img"][..., :3], atol=1e-1, rtol=1e-1)
        if expect_all:
            assert (r["n_contributors"] == 1).all()


def test_culling_and_empty_cases(oracle):
    pts, tets, cell = scene_util.small_scene(40, seed=4)
    # camera looking away: nothing visible, all ranges (0,0)
    tcam = scenes.make_tcam(scenes.look_at((0, 0, 3.0), (0, 0, 6.0)), 16, 16, 60.0, tile=4)
    pr = oracle.project(tets, pts, tcam)
    assert pr["tiles_touched"].sum() == 0
    idx, ranges = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], 4, 4)
    assert idx.size == 0 and not ranges.any()
    out, dist, nc = oracle.forward(idx, ranges, tets, pts, cell, tcam, np.full((16, 16, 2), 0.5, np.float32))
    assert not out.any() and not dist.any() and not nc.any()
    # planar tet is culled (|n.(v3-v0)| < 1e-3)
    flat = np.array([[0, 0, 0], [1, 0, 0], [0, 1, 0], [0.3, 0.3, 5e-4]], np.float32)
    tcam = scene_util.camera(eye=(0.2, 0.2, 2.0))
    pr = oracle.project(np.array([[0, 1, 2, 3]], np.int32), flat, tcam)
    assert pr["tiles_touched"][0] == 0 and not pr["circumcenter"].any()
    # NaN vertex is reported
    bad = pts.copy()
    bad[3, 1] = np.nan
    assert oracle.project(tets, bad, tcam)["nan_seen"]


def test_golden_fixture(oracle):
    g = np.load(GOLDEN)
    tcam = scene_util.camera(eye=tuple(g["eye"]), H=int(g["H"]), W=int(g["W"]), tile=int(g["tile"]),
                             fov=float(g["fov"]), min_t=float(g["min_t"]))
    r = oracle.render(g["indices"], g["vertices"], g["cell_values"], tcam, g["jitter"])
    for k in ("tiles_touched", "rect", "vs_tetra", "circumcenter"):
        np.testing.assert_array_equal(r["project"][k], g[k])
    np.testing.assert_array_equal(r["sorted_idx"], g["sorted_idx"])
    np.testing.assert_array_equal(r["tile_ranges"], g["tile_ranges"])
    np.testing.assert_array_equal(r["n_contributors"], g["n_contributors"])
    np.testing.assert_allclose(r["output_img"], g["output_img"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(r["distortion_img"], g["distortion_img"], rtol=1e-5, atol=1e-6)
    vg, cg = oracle.backward(r["sorted_idx"], r["tile_ranges"], g["indices"], g["vertices"], g["cell_values"], tcam,
                             g["jitter"], r["output_img"], r["distortion_img"], r["n_contributors"], g["g_img"],
                             g["g_dist"])
    np.testing.assert_allclose(vg, g["vertices_grad"], rtol=1e-4, atol=1e-4 * np.abs(g["vertices_grad"]).max())
    np.testing.assert_allclose(cg, g["cell_grad"], rtol=1e-4, atol=1e-4 * np.abs(g["cell_grad"]).max())


def test_circumspheres_against_reference_torch_geometry(oracle):
    """Projection-stage circumcentres and the fp64 sort depth against values the reference's own
    utils/topo_utils.py calculate_circumcenters_torch produced (tests/golden/make_topo_golden.py)."""
    here = os.path.join(os.path.dirname(__file__), "golden")
    g = np.load(os.path.join(here, "small_scene.npz"))
    t = np.load(os.path.join(here, "topo_circumspheres.npz"))
    vis = g["tiles_touched"] > 0
    err = np.abs(g["circumcenter"].astype(np.float64) - t["circumcenter"]).max(1) / t["radius"]
    assert err[vis].max() < 1e-6                      # the stage writes float32
    tets = g["vertices"][g["indices"]]
    for i in range(0, len(tets), 7):
        p, c = oracle.power_f64(tets[i], g["eye"])
        ref = ((g["eye"] - t["circumcenter"][i]) ** 2).sum() - t["radius"][i] ** 2
        assert abs(p - ref) <= 1e-12 * max(1.0, abs(ref))
        assert np.abs(c - t["circumcenter"][i]).max() <= 1e-12 * max(1.0, t["radius"][i])


def test_constant_color_backward_against_finite_differences(oracle):
    """The oracle's constant-colour backward pass (the reference's formulation, undo included) is the gradient of
    its forward pass when no pair is skipped (min_alpha = 0; the reference skips alpha < 1/255 in the backward pass
    only, which drops vertex-gradient terms that are not small), alphas stay away from 1 and the loss reads the
    image only; checked in float64."""
    pts, tets, cell = scene_util.small_scene(60, seed=2, mu=-0.5, sigma=0.4, zero_frac=0.0)
    rng = np.random.default_rng(4)
    rgbs = np.concatenate([rng.uniform(0.1, 0.9, (tets.shape[0], 3)), rng.uniform(0.8, 2.5, (tets.shape[0], 1))], 1)
    H = W = 12
    tcam = scene_util.camera(H=H, W=W, tile=4)
    pr = oracle.project(tets, pts, tcam)
    idx, ranges = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], tcam["grid_height"],
                                     tcam["grid_width"])
    v64, r64 = pts.astype(np.float64), rgbs.astype(np.float64)
    g_img = rng.normal(size=(H, W, 4))
    g_img[..., 3] *= 0.3

    def loss(v, r):
        out, _, _ = oracle.forward_constant_color_f64(idx, ranges, tets, v, r, tcam)
        return float((out * g_img).sum())

    out, dist, nc = oracle.forward_constant_color_f64(idx, ranges, tets, v64, r64, tcam)
    vg, rg = oracle.backward_constant_color(idx, ranges, tets, v64, r64, tcam, out, dist, nc, g_img,
                                            np.zeros((H, W, 4)), dtype=np.float64, min_alpha=0.0)
    assert np.abs(rg).max() > 0 and np.abs(vg).max() > 0
    # the reference's cut changes the result visibly (which is why the check above runs without it)
    vg_ref, rg_ref = oracle.backward_constant_color(idx, ranges, tets, v64, r64, tcam, out, dist, nc, g_img,
                                                    np.zeros((H, W, 4)), dtype=np.float64)
    assert np.abs(rg_ref - rg).max() < 0.05 * np.abs(rg).max()
    eps = 1e-6
    order = np.argsort(-np.abs(rg).sum(1))[:6]
    for t in order:
        for k in range(4):
            rp, rm = r64.copy(), r64.copy()
            rp[t, k] += eps
            rm[t, k] -= eps
            fd = (loss(v64, rp) - loss(v64, rm)) / (2 * eps)
            assert abs(fd - rg[t, k]) <= 1e-5 * max(1.0, abs(fd)), (t, k, fd, rg[t, k])
    vorder = np.argsort(-np.abs(vg).sum(1))[:5]
    for vi in vorder:
        for k in range(3):
            vp, vm = v64.copy(), v64.copy()
            vp[vi, k] += eps
            vm[vi, k] -= eps
            fd = (loss(vp, r64) - loss(vm, r64)) / (2 * eps)
            assert abs(fd - vg[vi, k]) <= 1e-4 * max(1.0, abs(fd)), (vi, k, fd, vg[vi, k])
