"""The bounds-checked build of the library (-DRM_BOUNDS_CHECK) on small and ragged cases.

compute-sanitizer is not available where these tests run, so memory safety of the data-dependent
indexing (list cursors, hit-list slots, ids read from lists, region and chunk tables) is checked by
a second build of the same sources in which every such index is compared with the extent of its
array before the access; a violation sets a status bit and skips the access.  The cases run in a
child process that loads that build through RM_B200_LIBRARY; the status word must stay 0.  One more
case hands the forward pass a tile range that ends past the declared end of the list (inside a
larger allocation, so nothing can fault) and expects the checker to report it.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import sys
    import numpy as np
    import torch
    sys.path.insert(0, {root!r})
    sys.path.insert(0, {tests!r})
    import scene_util
    from radiance_meshes_b200 import _lib, raster, scenes
    from radiance_meshes_b200.render import render, tcam_to_device
    from delaunay_rasterization.internal.render_err import tet_error_stats
    assert _lib.bounds_checked(), "the bounds-checked build was not loaded"
    dev = torch.device("cuda:0")

    def frame(pts, tets, cell, tcam, seed):
        H, W = tcam["image_height"], tcam["image_width"]
        v = torch.tensor(pts, device=dev, requires_grad=True)
        c = torch.tensor(cell, device=dev, requires_grad=True)
        idx = torch.tensor(tets, device=dev, dtype=torch.int32)
        t = tcam_to_device(tcam, dev)
        pkg = render(idx, v, c, t, torch.tensor(scene_util.jitter(H, W, seed), device=dev))
        (pkg["image"].sum() + 0.1 * pkg["distortion_img"].sum()).backward()
        tet_error_stats(pkg["sorted_tetra_idx"], pkg["tile_ranges"], idx, v.detach(), c.detach(), t,
                        torch.rand((H, W), device=dev), torch.rand((H, W), device=dev), pkg["mask"].to(torch.int32))
        torch.cuda.synchronize()
        return int(pkg["sorted_tetra_idx"].shape[0])

    total = 0
    pts, tets, cell = scene_util.small_scene(400, seed=3, zero_frac=0.3)
    for (H, W, tile) in [(64, 80, 4), (37, 53, 4), (30, 30, 5), (33, 20, 3), (48, 64, 8), (40, 40, 16)]:
        total += frame(pts, tets, cell, scene_util.camera(H=H, W=W, tile=tile), tile)
    # camera inside the mesh, dense scene with early termination, a view that sees nothing, one large grid
    total += frame(pts, tets, cell, scenes.make_tcam(scenes.look_at((0.05, 0.02, -0.1), (0.4, 0.1, 1.0)), 48, 48, 90.0,
                                                     tile=4, min_t=0.02), 7)
    p2, t2, c2 = scene_util.small_scene(1500, seed=9, mu=3.0, sigma=0.5, zero_frac=0.0)
    total += frame(p2, t2, c2, scene_util.camera(H=64, W=64, tile=4), 8)
    total += frame(pts, tets, cell, scenes.make_tcam(scenes.look_at((0, 0, 3.0), (0, 0, 6.0)), 16, 16, 60.0, tile=4), 9)
    total += frame(p2, t2, c2, scene_util.camera(H=270, W=480, tile=4), 10)
    status = _lib.bounds_status()
    print("CLEAN", total, status)

    # a tile range that ends past the declared end of the list: reported, and skipped
    tcam = scene_util.camera(H=32, W=32, tile=4)
    cam = raster.CameraArgs(tcam_to_device(tcam, dev), dev)
    v = torch.tensor(pts, device=dev)
    idx = torch.tensor(tets, device=dev, dtype=torch.int32)
    bctx = raster.project_and_bin(idx, v, tcam_to_device(tcam, dev))
    n, _ = raster.read_info(bctx)
    lists = raster.build_tile_lists(bctx, n)
    roomy = torch.zeros((n + 256,), dtype=torch.int32, device=dev)
    roomy[:n] = lists
    ranges = bctx["tile_ranges"].clone()
    last = int(torch.nonzero(ranges[:, 1] == n)[-1])
    ranges[last, 1] = n + 40
    recs = raster.pack_records(idx, v, torch.tensor(cell, device=dev), cam, bctx["tiles_touched"])
    raster.forward(roomy[:n], ranges, recs, cam, torch.full((32, 32, 2), 0.5, device=dev))
    torch.cuda.synchronize()
    print("CAUGHT", _lib.bounds_status())
""")


def test_bounds_checked_build_stays_clean(cuda_lib):
    from radiance_meshes_b200.csrc import build
    lib = build.build(variant="check")
    env = dict(os.environ, RM_B200_LIBRARY=lib)
    code = CHILD.format(root=ROOT, tests=os.path.join(ROOT, "tests"))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = {ln.split()[0]: ln.split()[1:] for ln in out.stdout.splitlines() if ln[:5] in ("CLEAN", "CAUGH")}
    assert int(lines["CLEAN"][0]) > 100_000          # the cases did walk lists
    assert int(lines["CLEAN"][1]) == 0, f"bounds violations, site bits {int(lines['CLEAN'][1]):#x}"
    assert int(lines["CAUGHT"][0]) & 1, "the checker missed a tile range past the end of the list"
