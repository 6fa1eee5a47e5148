"""Constant-colour debug renderer (forward) against the oracle, through the drop-in module."""
import numpy as np
import pytest
import torch

import scene_util
from radiance_meshes_b200 import scenes

pytestmark = pytest.mark.gpu


class _Camera:
    """The attributes render_constant_color reads from the reference's Camera (data/camera.py:72-91)."""

    def __init__(self, tcam):
        self.image_height, self.image_width = tcam["image_height"], tcam["image_width"]
        self._t = tcam

    def to_dict(self, device):
        keep = ("world_view_transform", "K", "cam_pos", "distortion_params", "image_height", "image_width",
                "camera_type", "fovy", "fovx")
        out = {}
        for k in keep:
            v = self._t[k]
            out[k] = torch.as_tensor(v, dtype=torch.float32).to(device) if isinstance(v, np.ndarray) else v
        return out


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


@pytest.mark.parametrize("tile", [16, 8, 4])
def test_render_constant_color_matches_oracle(oracle, cuda_lib, tile):
    from delaunay_rasterization.internal.alphablend_tiled_slang import AlphaBlendTiledRender, render_constant_color
    pts, tets, cell = scene_util.small_scene(500, seed=31, zero_frac=0.2)
    H, W = 72, 100
    tcam = scene_util.camera(H=H, W=W, tile=tile, min_t=0.1)
    rng = np.random.default_rng(4)
    rgbs = np.concatenate([rng.uniform(0, 1, (tets.shape[0], 3)), 3.0 * cell[:, :1]], axis=1).astype(np.float32)
    rgbs[::17, 3] = -0.5                                   # negative densities behave as empty
    dev = torch.device("cuda:0")
    idx = torch.tensor(tets, device=dev, dtype=torch.int32)
    v = torch.tensor(pts, device=dev)
    pkg = render_constant_color(idx, v, None, _Camera(tcam), cell_values=torch.tensor(rgbs, device=dev),
                                tile_size=tile, min_t=0.1)
    pr = oracle.project(tets, pts, tcam)
    ref_idx, ref_ranges = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], tcam["grid_height"],
                                             tcam["grid_width"])
    out, dist, nc = oracle.forward_constant_color(ref_idx, ref_ranges, tets, pts, rgbs, tcam)
    assert out[..., :3].max() > 0.1 and (out[..., 3] < 1 / 255).any() and (out[..., 3] > 0.5).any()
    got = pkg["render"].permute(1, 2, 0).cpu().numpy()
    assert rel_l2(got, out[..., :3]) <= 1e-4
    np.testing.assert_array_equal(pkg["mask"].cpu().numpy(), pr["tiles_touched"] > 0)
    # all four channels, the distortion moments and the contributor counts through the autograd function
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader
    from radiance_meshes_b200.render import tcam_to_device
    grid = RenderGrid(H, W, tile_height=tile, tile_width=tile)
    tdev = tcam_to_device(tcam, dev)
    sidx, ranges, *_ = vertex_and_tile_shader(idx, v, tdev, grid)
    with torch.no_grad():
        img, dimg = AlphaBlendTiledRender.apply(sidx, ranges, idx, v, torch.tensor(rgbs, device=dev), grid, tdev,
                                                100, -0.1)
    assert rel_l2(img.cpu().numpy(), out) <= 1e-4
    d_got = dimg.cpu().numpy()
    same_walk = np.isclose(img.cpu().numpy()[..., 3], out[..., 3], rtol=1e-3, atol=1e-6)
    assert same_walk.mean() > 0.999                          # a transmittance on the 1/255 cut-off may flip
    assert rel_l2(d_got[same_walk], dist[same_walk]) <= 1e-4


@pytest.mark.parametrize("tile", [16, 4])
def test_backward_against_oracle(oracle, cuda_lib, tile):
    """Gradients of the constant-colour renderer (vertices and rgbs) against the oracle's restatement of the
    reference's backward pass, upstream gradients on the image and on the distortion moments."""
    from delaunay_rasterization.internal.alphablend_tiled_slang import AlphaBlendTiledRender
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader
    from radiance_meshes_b200.render import tcam_to_device
    pts, tets, cell = scene_util.small_scene(300, seed=12, zero_frac=0.2)
    H, W = 48, 64
    tcam = scene_util.camera(H=H, W=W, tile=tile)
    rng = np.random.default_rng(8)
    rgbs = np.concatenate([rng.uniform(0, 1, (tets.shape[0], 3)), 2.0 * cell[:, :1]], axis=1).astype(np.float32)
    g_img = rng.normal(size=(H, W, 4)).astype(np.float32)
    g_dist = (1e-3 * rng.normal(size=(H, W, 4))).astype(np.float32)
    dev = torch.device("cuda:0")
    idx = torch.tensor(tets, device=dev, dtype=torch.int32)
    v = torch.tensor(pts, device=dev, requires_grad=True)
    r = torch.tensor(rgbs, device=dev, requires_grad=True)
    grid = RenderGrid(H, W, tile_height=tile, tile_width=tile)
    tdev = tcam_to_device(tcam, dev)
    sidx, ranges, *_ = vertex_and_tile_shader(idx, v.detach(), tdev, grid)
    img, dimg = AlphaBlendTiledRender.apply(sidx, ranges, idx, v, r, grid, tdev, 100, -0.1)
    ((img * torch.tensor(g_img, device=dev)).sum() + (dimg * torch.tensor(g_dist, device=dev)).sum()).backward()
    pr = oracle.project(tets, pts, tcam)
    ref_idx, ref_ranges = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], tcam["grid_height"],
                                             tcam["grid_width"])
    out, dist, nc = oracle.forward_constant_color(ref_idx, ref_ranges, tets, pts, rgbs, tcam)
    vg, rg = oracle.backward_constant_color(ref_idx, ref_ranges, tets, pts, rgbs, tcam, out, dist, nc, g_img, g_dist)
    assert np.abs(vg).max() > 0 and np.abs(rg).max() > 0
    assert rel_l2(r.grad.cpu().numpy(), rg) <= 1e-3
    assert rel_l2(v.grad.cpu().numpy(), vg) <= 1e-3
