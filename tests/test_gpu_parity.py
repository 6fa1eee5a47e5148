"""GPU parity tests: every stage of the CUDA path, called through the C ABI
(via the drop-in delaunay_rasterization entry points), against the CPU oracle on
the same seeded inputs.

Gates: tile lists, rectangles, counts, sort depths bit-exact; images and
distortion moments within 1e-4 relative L2 (fp32); gradients within 1e-3
relative L2.
"""
import os

import numpy as np
import pytest
import torch

import scene_util
from radiance_meshes_b200 import scenes

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "small_scene.npz")
IMG_TOL = 1e-4
GRAD_TOL = 1e-3


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def gpu_render(pts, tets, cell, tcam, jit, g_img=None, g_dist=None):
    from radiance_meshes_b200.render import render, tcam_to_device
    dev = torch.device("cuda:0")
    v = torch.tensor(pts, device=dev, requires_grad=True)
    c = torch.tensor(cell, device=dev, requires_grad=True)
    idx = torch.tensor(tets, device=dev, dtype=torch.int32)
    j = torch.tensor(jit, device=dev)
    pkg = render(idx, v, c, tcam_to_device(tcam, dev), j)
    out = {k: pkg[k].detach().cpu().numpy() for k in ("image", "distortion_img", "sorted_tetra_idx", "tile_ranges",
                                                       "vs_tetra", "circumcenter", "rect", "mask")}
    if g_img is not None:
        loss = (pkg["image"] * torch.tensor(g_img, device=dev)).sum() + \
               (pkg["distortion_img"] * torch.tensor(g_dist, device=dev)).sum()
        loss.backward()
        out["vertices_grad"] = v.grad.cpu().numpy()
        out["cell_grad"] = c.grad.cpu().numpy()
    return out


def check_against_oracle(oracle, pts, tets, cell, tcam, jit, seed=0, check_grad=True, max_flips=0.01):
    """All stages against the oracle.

    The image is compared on every pixel.  The distortion moments and the
    gradients are compared with the rounding-decided pixels of the reference
    algorithm masked out (oracle.sensitive_pixels: grazing ray/tet contacts add a
    tet's whole density to the moments or nothing; a log-transmittance on the
    -5.5 cut-off walks one more tet or not).  On the masked pixels the two sides
    may legitimately differ; the share of pixels that actually do is bounded.
    """
    H, W = tcam["image_height"], tcam["image_width"]
    rng = np.random.default_rng(seed)
    ref = oracle.render(tets, pts, cell, tcam, jit)
    keep = ~oracle.sensitive_pixels(ref["sorted_idx"], ref["tile_ranges"], tets, pts, cell, tcam, jit, tol=2e-5)
    g_img = (rng.normal(size=(H, W, 4)) * keep[..., None]).astype(np.float32)
    g_dist = (0.05 * rng.normal(size=(H, W, 5)) * keep[..., None]).astype(np.float32)
    got = gpu_render(pts, tets, cell, tcam, jit, g_img if check_grad else None, g_dist)
    # --- bit-exact integer / index work
    np.testing.assert_array_equal(got["rect"], ref["project"]["rect"])
    np.testing.assert_array_equal(got["mask"], ref["project"]["tiles_touched"] > 0)
    np.testing.assert_array_equal(got["vs_tetra"].view(np.uint32), ref["project"]["vs_tetra"].view(np.uint32))
    np.testing.assert_array_equal(got["circumcenter"].view(np.uint32),
                                  ref["project"]["circumcenter"].view(np.uint32))
    np.testing.assert_array_equal(got["tile_ranges"], ref["tile_ranges"])
    np.testing.assert_array_equal(got["sorted_tetra_idx"], ref["sorted_idx"])
    # --- floating point within tolerance
    if ref["output_img"].any():
        assert rel_l2(got["image"], ref["output_img"]) <= IMG_TOL
        assert rel_l2(got["distortion_img"][keep], ref["distortion_img"][keep]) <= IMG_TOL
        diff = np.abs(got["distortion_img"] - ref["distortion_img"]).max(-1)
        flips = diff > 1e-3 * (np.abs(ref["distortion_img"]).max(-1) + 1e-6)
        assert not (flips & keep).any()
        assert flips.mean() <= max_flips
    else:
        assert not got["image"].any()
    if check_grad:
        vg, cg = oracle.backward(ref["sorted_idx"], ref["tile_ranges"], tets, pts, cell, tcam, jit,
                                 ref["output_img"], ref["distortion_img"], ref["n_contributors"], g_img, g_dist)
        if np.abs(vg).max() > 0:
            assert rel_l2(got["vertices_grad"], vg) <= GRAD_TOL
            assert rel_l2(got["cell_grad"], cg) <= GRAD_TOL
        else:
            assert not got["vertices_grad"].any() and not got["cell_grad"].any()
    return ref, got


@pytest.mark.parametrize("tile", [4, 8, 16])
def test_small_scene_all_stages(oracle, cuda_lib, tile):
    pts, tets, cell = scene_util.small_scene(300, seed=tile)
    H, W = 64, 80
    tcam = scene_util.camera(H=H, W=W, tile=tile)
    check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, 1))


def test_ragged_image_and_odd_tile(oracle, cuda_lib):
    # image not a multiple of the tile; tile sizes that are not multiples of 4
    pts, tets, cell = scene_util.small_scene(200, seed=21)
    for (H, W, tile) in [(37, 53, 4), (30, 30, 5), (33, 20, 3)]:
        tcam = scene_util.camera(H=H, W=W, tile=tile)
        check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, 2))


def test_camera_inside_mesh(oracle, cuda_lib):
    pts, tets, cell = scene_util.small_scene(400, seed=5, zero_frac=0.4)
    H = W = 48
    tcam = scenes.make_tcam(scenes.look_at((0.05, 0.02, -0.1), (0.4, 0.1, 1.0)), H, W, 90.0, tile=4, min_t=0.02)
    check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, 3))


def test_config1_cpu_runnable_reference_case(oracle, cuda_lib):
    # 2,000 points uniform in [-1,1]^3, 128x128, fov 60, eye at distance 3
    sc = scenes.make_scene(1)
    tcam = scenes.config_camera(1)
    ref, got = check_against_oracle(oracle, sc["vertices"], sc["indices"], sc["cell_values"], tcam,
                                    np.full((128, 128, 2), 0.5, np.float32))
    assert ref["sorted_idx"].shape[0] > 100_000


def test_dense_scene_early_termination(oracle, cuda_lib):
    # high densities: most pixels terminate early, exercising the per-tile fetch stop
    pts, tets, cell = scene_util.small_scene(2000, seed=9, mu=3.0, sigma=0.5, zero_frac=0.0)
    H = W = 64
    tcam = scene_util.camera(H=H, W=W, tile=4)
    ref, got = check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, 4))
    assert ref["output_img"][..., 3].min() < -5.5


def test_empty_and_culled(oracle, cuda_lib):
    pts, tets, cell = scene_util.small_scene(40, seed=4)
    # looking away: N = 0
    tcam = scenes.make_tcam(scenes.look_at((0, 0, 3.0), (0, 0, 6.0)), 16, 16, 60.0, tile=4)
    check_against_oracle(oracle, pts, tets, cell, tcam, np.full((16, 16, 2), 0.5, np.float32))
    # a planar tet next to a regular one
    v = np.array([[0, 0, 0], [1, 0, 0], [0, 1, 0], [0.3, 0.3, 5e-4], [0.2, 0.2, 0.8]], np.float32)
    t = np.array([[0, 1, 2, 3], [0, 1, 2, 4]], np.int32)
    c = np.array([[1.0, .5, .5, .5, 0, 0, 0], [2.0, .2, .4, .6, .1, -.1, .2]], np.float32)
    tcam = scene_util.camera(eye=(0.2, 0.2, 2.5), H=32, W=32)
    check_against_oracle(oracle, v, t, c, tcam, np.full((32, 32, 2), 0.5, np.float32))


def test_nan_vertices_raise(cuda_lib):
    from radiance_meshes_b200.render import render, tcam_to_device
    pts, tets, cell = scene_util.small_scene(40, seed=4)
    pts[7, 2] = np.nan
    dev = torch.device("cuda:0")
    tcam = tcam_to_device(scene_util.camera(H=16, W=16), dev)
    with pytest.raises(AssertionError, match="NaN"):
        render(torch.tensor(tets, device=dev), torch.tensor(pts, device=dev), torch.tensor(cell, device=dev), tcam)


def test_golden_fixture(cuda_lib):
    g = np.load(GOLDEN)
    tcam = scene_util.camera(eye=tuple(g["eye"]), H=int(g["H"]), W=int(g["W"]), tile=int(g["tile"]),
                             fov=float(g["fov"]), min_t=float(g["min_t"]))
    got = gpu_render(g["vertices"], g["indices"], g["cell_values"], tcam, g["jitter"], g["g_img"], g["g_dist"])
    np.testing.assert_array_equal(got["rect"], g["rect"])
    np.testing.assert_array_equal(got["sorted_tetra_idx"], g["sorted_idx"])
    np.testing.assert_array_equal(got["tile_ranges"], g["tile_ranges"])
    np.testing.assert_array_equal(got["vs_tetra"], g["vs_tetra"])
    assert rel_l2(got["image"], g["output_img"]) <= IMG_TOL
    assert rel_l2(got["distortion_img"], g["distortion_img"]) <= IMG_TOL
    assert rel_l2(got["vertices_grad"], g["vertices_grad"]) <= GRAD_TOL
    assert rel_l2(got["cell_grad"], g["cell_grad"]) <= GRAD_TOL


def test_vertex_stage_backward(oracle, cuda_lib):
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader
    from radiance_meshes_b200.render import tcam_to_device
    pts, tets, cell = scene_util.small_scene(300, seed=13)
    tcam = scene_util.camera(H=32, W=32)
    dev = torch.device("cuda:0")
    v = torch.tensor(pts, device=dev, requires_grad=True)
    grid = RenderGrid(32, 32, tile_width=4, tile_height=4)
    _, _, vs_tetra, circumcenter, mask, _ = vertex_and_tile_shader(torch.tensor(tets, device=dev), v,
                                                                   tcam_to_device(tcam, dev), grid)
    rng = np.random.default_rng(0)
    g_vs = rng.normal(size=vs_tetra.shape).astype(np.float32)
    g_cc = rng.normal(size=circumcenter.shape).astype(np.float32)
    ((vs_tetra * torch.tensor(g_vs, device=dev)).sum() + (circumcenter * torch.tensor(g_cc, device=dev)).sum()
     ).backward()
    pr = oracle.project(tets, pts, tcam)
    ref = oracle.vertex_backward(tets, pts, tcam, pr["tiles_touched"], g_vs, g_cc)
    assert rel_l2(v.grad.cpu().numpy(), ref) <= GRAD_TOL


def test_medium_scene_sort_classes(oracle, cuda_lib):
    # 20k points at 256x256 with 16x16 tiles: tile lists of several thousand entries,
    # exercising the large shared-memory sort class
    pts = scenes.points_gaussians(20_000, seed=3)
    tets = scenes.delaunay(pts)
    cell = scenes._features(np.random.default_rng(3), tets.shape[0], -1.0, 1.5, 0.3)
    H = W = 256
    tcam = scenes.make_tcam(scenes.look_at((0.0, 0.3, 3.2)), H, W, 50.0, tile=16, min_t=0.1)
    ref, got = check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, 7), check_grad=True)
    lens = ref["tile_ranges"][:, 1] - ref["tile_ranges"][:, 0]
    assert lens.max() > 2048


def test_tile_row_bands_match_full_frame(oracle, cuda_lib):
    # one frame rendered as two tile-row bands (the multi-GPU split of a large
    # frame) equals the full-frame render: lists are the corresponding subsets,
    # image rows are identical
    from radiance_meshes_b200 import dist as rmdist
    from radiance_meshes_b200.render import render, tcam_to_device
    pts, tets, cell = scene_util.small_scene(500, seed=23)
    H, W = 72, 64
    tcam_np = scene_util.camera(H=H, W=W, tile=4)
    dev = torch.device("cuda:0")
    idx_t = torch.tensor(tets, device=dev)
    v = torch.tensor(pts, device=dev)
    c = torch.tensor(cell, device=dev)
    jit = torch.tensor(scene_util.jitter(H, W, 9), device=dev)
    full = render(idx_t, v, c, tcam_to_device(tcam_np, dev), jit)
    gw, gh = tcam_np["grid_width"], tcam_np["grid_height"]
    weights = rmdist.row_weights_from_rects(full["rect"], full["mask"].int(), gh)
    lens = (full["tile_ranges"][:, 1] - full["tile_ranges"][:, 0]).reshape(gh, gw).sum(1)
    assert torch.equal(weights.cpu(), lens.cpu().long())
    bands = rmdist.tile_row_bands(gh, 2, weights.cpu().numpy())
    combined = torch.zeros_like(full["image"])
    combined_dist = torch.zeros_like(full["distortion_img"])
    for band in bands:
        tcam_b = dict(tcam_to_device(tcam_np, dev), tile_rows=band)
        part = render(idx_t, v, c, tcam_b, jit)
        y0, y1 = band[0] * 4, min(band[1] * 4, H)
        combined[y0:y1] = part["image"][y0:y1]
        combined_dist[y0:y1] = part["distortion_img"][y0:y1]
        fr, pr = full["tile_ranges"].cpu().numpy(), part["tile_ranges"].cpu().numpy()
        fi, pi = full["sorted_tetra_idx"].cpu().numpy(), part["sorted_tetra_idx"].cpu().numpy()
        for t in range(band[0] * gw, band[1] * gw):
            np.testing.assert_array_equal(pi[pr[t, 0]:pr[t, 1]], fi[fr[t, 0]:fr[t, 1]])
        outside = np.ones(gh * gw, bool)
        outside[band[0] * gw:band[1] * gw] = False
        assert not pr[outside].any()
    assert torch.equal(combined, full["image"])
    assert torch.equal(combined_dist, full["distortion_img"])


def test_distorted_perspective_camera(oracle, cuda_lib):
    # radial + tangential distortion: 3 samples per clipped edge in the extent search,
    # Newton undistortion in the ray generation; only + - * / are involved, so the
    # tile lists stay bit-exact
    pts, tets, cell = scene_util.small_scene(300, seed=41)
    H, W = 48, 56
    tcam = scene_util.camera(H=H, W=W, tile=4, distortion=[0.08, -0.02, 0.003, -0.002])
    check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, 11))


def test_fisheye_camera(oracle, cuda_lib):
    # fisheye projection: acos/sin are evaluated as the same fixed double-precision series on both
    # sides, so rectangles and tile lists are bit-exact like the pinhole ones; image and gradients
    # within the usual tolerances (the ray directions use the fast sine/cosine)
    pts, tets, cell = scene_util.small_scene(300, seed=43)
    H, W = 48, 48
    for fov, dist in ((100.0, None), (140.0, (0.02, -0.01, 0.001, 0.002))):
        tcam = scene_util.camera(H=H, W=W, tile=4, fov=fov, camera_type=1, distortion=dist)
        ref, got = check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, 12))
        assert ref["sorted_idx"].shape[0] > 1000


def test_densification_statistics(oracle, cuda_lib):
    # calc_tet_err: per-tet error moments and hit counts against the oracle
    from delaunay_rasterization.internal.render_err import tet_error_stats
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader
    from radiance_meshes_b200.render import tcam_to_device
    pts, tets, cell = scene_util.small_scene(600, seed=29, zero_frac=0.3)
    H, W = 64, 72
    tcam_np = scene_util.camera(H=H, W=W, tile=4)
    rng = np.random.default_rng(3)
    pixel_err = rng.normal(0, 0.1, (H, W)).astype(np.float32)
    ssim_err = rng.uniform(0, 1, (H, W)).astype(np.float32)
    ref = oracle.render(tets, pts, cell, tcam_np)
    err_ref, cnt_ref = oracle.tet_err(ref["sorted_idx"], ref["tile_ranges"], tets, pts, cell, tcam_np, pixel_err,
                                      ssim_err)
    dev = torch.device("cuda:0")
    tcam = tcam_to_device(tcam_np, dev)
    idx_t, v, c = torch.tensor(tets, device=dev), torch.tensor(pts, device=dev), torch.tensor(cell, device=dev)
    grid = RenderGrid(H, W, tile_width=4, tile_height=4)
    sorted_idx, ranges, _, _, mask, _ = vertex_and_tile_shader(idx_t, v, tcam, grid)
    np.testing.assert_array_equal(sorted_idx.cpu().numpy(), ref["sorted_idx"])
    err, cnt = tet_error_stats(sorted_idx, ranges, idx_t, v, c, tcam, torch.tensor(pixel_err, device=dev),
                               torch.tensor(ssim_err, device=dev), mask.to(torch.int32))
    err, cnt = err.cpu().numpy(), cnt.cpu().numpy()
    assert cnt_ref[:, 0].sum() > 10_000
    assert not err[:, 3:5].any()
    # sums of fp32 products in a different order, plus a handful of rounding-decided hits
    assert rel_l2(err, err_ref) <= 1e-3
    dcount = np.abs(cnt[:, 0] - cnt_ref[:, 0])
    assert dcount.max() <= 2 and (dcount > 0).mean() <= 0.01
    same = dcount == 0
    assert np.abs(cnt[same, 1] - cnt_ref[same, 1]).max() <= 2 + 1e-4 * cnt_ref[:, 1].max()


def test_host_frame_pipeline_matches_direct_path():
    """Host buffers in / host buffers out with overlapped copies gives the same frame and gradients."""
    import torch
    from radiance_meshes_b200.render import HostFramePipeline, render, tcam_to_device
    pts, tets, cell = scene_util.small_scene(400, seed=21)
    sc = dict(indices=np.ascontiguousarray(tets, np.int32), vertices=pts, cell_values=cell)
    tcam_np = scene_util.camera(H=96, W=128, tile=4)
    dev = torch.device("cuda:0")
    tcam = tcam_to_device(tcam_np, dev)
    rng = np.random.default_rng(5)
    H, W = tcam_np["image_height"], tcam_np["image_width"]
    host = dict(indices=torch.from_numpy(sc["indices"]).pin_memory(),
                vertices=torch.from_numpy(sc["vertices"]).pin_memory(),
                cell=torch.from_numpy(sc["cell_values"]).pin_memory(),
                jitter=torch.from_numpy(rng.uniform(0, 1, (H, W, 2)).astype(np.float32)).pin_memory(),
                g_img=torch.from_numpy(rng.normal(size=(H, W, 4)).astype(np.float32)).pin_memory(),
                g_dist=torch.from_numpy((0.01 * rng.normal(size=(H, W, 5))).astype(np.float32)).pin_memory())
    T, V = sc["indices"].shape[0], sc["vertices"].shape[0]
    out = dict(image=torch.empty((H, W, 4)).pin_memory(), dist=torch.empty((H, W, 5)).pin_memory(),
               vg=torch.empty((V, 3)).pin_memory(), cg=torch.empty((T, 7)).pin_memory())
    pipe = HostFramePipeline(dev)
    for _ in range(3):          # staging buffers are reused from the second frame on
        for t in out.values():
            t.fill_(float("nan"))
        pipe.step(host, out, tcam)
    # two frames in flight, each with its own result buffers
    outs = [out, {k: torch.empty_like(t).pin_memory() for k, t in out.items()}]
    pipe2 = HostFramePipeline(dev, frames_in_flight=2)
    tickets = []
    for i in range(5):
        if i >= 2:
            pipe2.wait(tickets[i - 2])
        for t in outs[i % 2].values():
            t.fill_(float("nan"))
        tickets.append(pipe2.submit(host, outs[i % 2], tcam))
    pipe2.wait(tickets[-2])
    pipe2.wait(tickets[-1])
    torch.cuda.synchronize()
    for k in ("image", "dist"):
        assert torch.equal(outs[0][k], outs[1][k])
    d = {k: v.to(dev) for k, v in host.items()}
    v = d["vertices"].requires_grad_(True)
    c = d["cell"].requires_grad_(True)
    pkg = render(d["indices"], v, c, tcam, d["jitter"])
    torch.autograd.backward([pkg["image"], pkg["distortion_img"]], [d["g_img"], d["g_dist"]])
    assert torch.equal(out["image"], pkg["image"].detach().cpu())
    assert torch.equal(out["dist"], pkg["distortion_img"].detach().cpu())
    for got, want in ((out["vg"], v.grad.cpu()), (out["cg"], c.grad.cpu()), (outs[1]["vg"], v.grad.cpu()),
                      (outs[1]["cg"], c.grad.cpu())):   # float atomics: order varies
        assert torch.isfinite(got).all()
        assert float((got - want).norm() / want.norm().clamp_min(1e-20)) < 1e-5


@pytest.mark.parametrize("H,W,tile,npts", [(1080, 1920, 4, 30_000),     # 4080 regions: two-pass region sort
                                           (2160, 3840, 2, 4_000),      # 64800 regions: above the shared-memory table
                                           (40, 2056, 4, 3_000)])       # one region row, ragged right edge
def test_large_grid_tile_lists_bit_exact(oracle, cuda_lib, H, W, tile, npts):
    """Tile lists on grids large enough for every region-sort configuration, against the oracle's
    stable sort of (tile, depth) keys (projection + lists only: no pixels are rendered)."""
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader
    from radiance_meshes_b200.render import tcam_to_device
    pts = scenes.points_gaussians(npts, seed=11)
    tets = scenes.delaunay(pts)
    tcam = scenes.make_tcam(scenes.look_at((0.2, 0.1, 2.6)), H, W, 60.0, tile=tile, min_t=0.1)
    pr = oracle.project(tets, pts, tcam)
    ref_idx, ref_ranges = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"],
                                             tcam["grid_height"], tcam["grid_width"])
    dev = torch.device("cuda:0")
    grid = RenderGrid(H, W, tile_height=tile, tile_width=tile)
    idx, ranges, vs, cc, mask, rect = vertex_and_tile_shader(
        torch.tensor(tets, device=dev, dtype=torch.int32), torch.tensor(pts, device=dev), tcam_to_device(tcam, dev),
        grid)
    np.testing.assert_array_equal(rect.cpu().numpy(), pr["rect"])
    np.testing.assert_array_equal(ranges.cpu().numpy(), ref_ranges)
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx)
    assert len(ref_idx) > 10_000


def test_full_size_lists_properties(cuda_lib):
    """At the benchmark's size (1M points would take a minute to triangulate: 200k here, same 1080p grid)
    the lists are checked through properties: every tile's segment is ascending in (depth bits, tet id),
    holds exactly the tets whose rectangle covers the tile, and the segments tile the array."""
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader
    from radiance_meshes_b200.render import tcam_to_device
    pts = scenes.points_gaussians(200_000, seed=5)
    tets = scenes.delaunay(pts)
    H, W, tile = 1080, 1920, 4
    tcam = scenes.make_tcam(scenes.look_at((0.0, 0.4, 2.8)), H, W, 60.0, tile=tile, min_t=0.1)
    dev = torch.device("cuda:0")
    grid = RenderGrid(H, W, tile_height=tile, tile_width=tile)
    idx, ranges, vs, cc, mask, rect = vertex_and_tile_shader(
        torch.tensor(tets, device=dev, dtype=torch.int32), torch.tensor(pts, device=dev), tcam_to_device(tcam, dev),
        grid)
    N = idx.shape[0]
    gw = grid.grid_width
    lens = (ranges[:, 1] - ranges[:, 0]).long()
    assert int(lens.sum()) == N and N > 5_000_000
    nonempty = lens > 0
    starts = ranges[:, 0].long()[nonempty]
    assert torch.equal(starts, (torch.cumsum(lens[nonempty], 0) - lens[nonempty]))        # segments tile the array
    tile_of = torch.repeat_interleave(torch.arange(ranges.shape[0], device=dev), lens)   # tile of every entry
    t = idx.long()
    r = rect[t].long()
    tx, ty = tile_of % gw, tile_of // gw
    assert bool(((tx >= r[:, 0]) & (tx < r[:, 2]) & (ty >= r[:, 1]) & (ty < r[:, 3])).all())   # only covering tets
    area = ((rect[:, 2] - rect[:, 0]) * (rect[:, 3] - rect[:, 1])).long()
    assert int(area[mask].sum()) == N                                                          # and all of them
    # ascending (sortable depth bits, tet id) inside every tile
    bits = vs[:, 2].contiguous().view(torch.int32).long() & 0xFFFFFFFF
    key = torch.where(bits >> 31 == 1, (~bits) & 0xFFFFFFFF, bits | 0x80000000)
    k = key[t] * (1 << 23) + t                      # 32 key bits above 23 id bits (ids < 2^23 here)
    assert tets.shape[0] < (1 << 23)
    same_tile = tile_of[1:] == tile_of[:-1]
    assert bool((k[1:][same_tile] > k[:-1][same_tile]).all())


def test_config2_forward_only_case(oracle, cuda_lib):
    # 100,000 points from 8 Gaussians -> ~673k tets, 800x800, fov 50, forward only: every stage against
    # the oracle at the full size of the configuration
    sc = scenes.make_scene(2)
    tcam = scenes.config_camera(2)
    H, W = tcam["image_height"], tcam["image_width"]
    assert (H, W) == (800, 800) and sc["indices"].shape[0] > 600_000
    ref, got = check_against_oracle(oracle, sc["vertices"], sc["indices"], sc["cell_values"], tcam,
                                    scene_util.jitter(H, W, 2), check_grad=False)
    assert ref["sorted_idx"].shape[0] > 5_000_000


def test_config3_shaped_scene_fwd_bwd(oracle, cuda_lib):
    # the benchmark's scene law (clusters + far shell, 40 % empty tets) and ring camera at a size the
    # oracle renders in seconds: 60,000 points, 480x270
    sc = scenes.make_scene(3, n_points=60_000)
    tcam = scenes.config_camera(3, view=5, height=270, width=480)
    ref, got = check_against_oracle(oracle, sc["vertices"], sc["indices"], sc["cell_values"], tcam,
                                    scene_util.jitter(270, 480, 9), check_grad=True)
    assert ref["sorted_idx"].shape[0] > 1_000_000


@pytest.mark.parametrize("seed", list(range(8)))
def test_random_configurations(oracle, cuda_lib, seed):
    """Seeded sweep over image sizes, tile shapes, camera placements and densities: every stage against the
    oracle.  Exercises ragged tiles, non-square tiles, several 16-pixel groups per tile, regions cut by the
    image border and cameras inside the mesh."""
    rng = np.random.default_rng(1000 + seed)
    H, W = int(rng.integers(17, 140)), int(rng.integers(17, 180))
    th, tw = [(2, 2), (4, 4), (8, 8), (16, 16), (4, 8), (8, 4), (2, 16), (5, 3)][seed]
    n_points = int(rng.integers(80, 700))
    pts, tets, cell = scene_util.small_scene(n_points, seed=50 + seed, zero_frac=float(rng.uniform(0.0, 0.6)),
                                             sigma=float(rng.uniform(0.5, 2.0)))
    r = float(rng.uniform(0.2, 3.0))                       # below ~1: the camera sits inside the point cloud
    ang = rng.uniform(0, 2 * np.pi, 2)
    eye = (r * np.cos(ang[0]) * np.cos(ang[1]), r * np.sin(ang[1]), r * np.sin(ang[0]) * np.cos(ang[1]))
    tcam = scenes.make_tcam(scenes.look_at(eye), H, W, float(rng.uniform(35, 100)), tile=(th, tw),
                            min_t=float(rng.uniform(0.01, 0.3)))
    check_against_oracle(oracle, pts, tets, cell, tcam, scene_util.jitter(H, W, seed), seed=seed, check_grad=True,
                         max_flips=0.02)


def test_chunked_finish_hands_over_final_gradients(oracle, cuda_lib):
    """The backward pass split into ranges of tets (the form a multi-GPU job uses to sum finished ranges
    while the next one is computed) gives the same gradients, and every range is final when handed over."""
    from radiance_meshes_b200 import raster
    pts, tets, cell = scene_util.small_scene(1500, seed=33)
    assert tets.shape[0] >= 4096
    H, W = 64, 64
    tcam = scene_util.camera(H=H, W=W, tile=4)
    jit = scene_util.jitter(H, W, 6)
    rng = np.random.default_rng(2)
    g_img = rng.normal(size=(H, W, 4)).astype(np.float32)
    g_dist = (0.05 * rng.normal(size=(H, W, 5))).astype(np.float32)
    base = gpu_render(pts, tets, cell, tcam, jit, g_img, g_dist)

    class Sink:
        def __init__(self):
            self.seen, self.finished = [], False

        def __call__(self, t):
            self.seen.append((tuple(t.shape), t.clone()))

        def done(self):
            self.finished = True

    sink = Sink()
    raster.set_gradient_sink(sink, chunks=3)
    try:
        got = gpu_render(pts, tets, cell, tcam, jit, g_img, g_dist)
    finally:
        raster.set_gradient_sink(None)
    assert sink.finished and len(sink.seen) == 4 and sink.seen[-1][0] == (pts.shape[0], 3)
    assert sum(s[0][0] for s in sink.seen[:-1]) == tets.shape[0]
    cg_parts = torch.cat([s[1] for s in sink.seen[:-1]]).cpu().numpy()
    np.testing.assert_array_equal(cg_parts, got["cell_grad"])          # ranges were final when handed over
    np.testing.assert_array_equal(sink.seen[-1][1].cpu().numpy(), got["vertices_grad"])
    assert rel_l2(got["cell_grad"], base["cell_grad"]) <= 1e-5          # same sums up to the order of atomics
    assert rel_l2(got["vertices_grad"], base["vertices_grad"]) <= 1e-5
