"""render_err() end to end (delaunay_rasterization/internal/render_err.py:33-159 of the reference):
the drop-in function is driven the way utils/densification.py:137-238 drives it, with a stand-in
model, a stand-in camera and a stand-in `utils.ssim` module (the reference's own SSIM lives outside
this package), and its outputs are compared with the CPU oracle fed the same per-pixel errors."""
import sys
import types

import numpy as np
import pytest
import torch

import scene_util

pytestmark = pytest.mark.gpu


class _Camera:
    """The attributes render_err touches: image size, to_dict(device), gt_alpha_mask."""

    def __init__(self, tcam_np, alpha_mask):
        self.t = tcam_np
        self.image_height, self.image_width = tcam_np["image_height"], tcam_np["image_width"]
        self.gt_alpha_mask = alpha_mask

    def to_dict(self, device):
        keys = ("world_view_transform", "cam_pos", "K", "distortion_params")
        d = {k: torch.as_tensor(self.t[k], dtype=torch.float32).to(device) for k in keys}
        d.update({k: self.t[k] for k in ("image_height", "image_width", "fovy", "fovx", "camera_type")})
        return d


class _Model:
    feature_dim = 7

    def __init__(self, pts, tets, cell, device):
        self.device = device
        self.vertices = torch.tensor(pts, device=device)
        self.indices = torch.tensor(tets, device=device, dtype=torch.int32)
        self.cell = torch.tensor(cell, device=device)
        self.calls = 0

    def get_cell_values(self, camera, mask=None, all_circumcenters=None):
        self.calls += 1
        return None, (self.cell if mask is None else self.cell[mask])


def _ssim_stand_in(a, b):
    """[3,H,W] similarity map in [0,1]; any deterministic per-pixel function will do for the plumbing."""
    return 1.0 / (1.0 + 25.0 * (a - b) ** 2)


def test_render_err_end_to_end(oracle, cuda_lib, monkeypatch):
    utils_pkg = types.ModuleType("utils")
    ssim_mod = types.ModuleType("utils.ssim")
    ssim_mod.ssim = _ssim_stand_in
    utils_pkg.ssim = ssim_mod
    monkeypatch.setitem(sys.modules, "utils", utils_pkg)
    monkeypatch.setitem(sys.modules, "utils.ssim", ssim_mod)
    from delaunay_rasterization.internal.render_err import render_err

    dev = torch.device("cuda:0")
    pts, tets, cell = scene_util.small_scene(500, seed=31, zero_frac=0.3)
    H, W, tile = 60, 76, 4
    tcam_np = scene_util.camera(H=H, W=W, tile=tile)
    rng = np.random.default_rng(9)
    gt = rng.uniform(0, 1, (3, H, W)).astype(np.float32)
    alpha = (rng.uniform(0, 1, (1, H, W)) > 0.2).astype(np.float32)
    model = _Model(pts, tets, cell, dev)
    camera = _Camera(tcam_np, torch.tensor(alpha))
    tet_err, extras = render_err(torch.tensor(gt, device=dev), camera, model, tile_size=tile, min_t=tcam_np["min_t"])
    assert model.calls == 1
    assert tet_err.shape == (tets.shape[0], 16) and extras["tet_count"].shape == (tets.shape[0], 2)
    assert set(extras) == {"tet_count", "pixel_err", "ssim_err", "render_img", "cell_values"}

    # the same quantities on the CPU: oracle image -> the reference's error definitions -> oracle statistics
    ref = oracle.render(tets, pts, cell, tcam_np)
    img = np.clip(ref["output_img"][..., :3].transpose(2, 0, 1), 0, 1)
    l1 = (img - gt).mean(0) * alpha[0]
    ss = np.clip(1 - (1.0 / (1.0 + 25.0 * (img - gt) ** 2)).mean(0), 0, 1) * alpha[0]
    np.testing.assert_allclose(extras["pixel_err"].cpu().numpy(), l1, atol=2e-5)
    np.testing.assert_allclose(extras["ssim_err"].cpu().numpy(), ss, atol=2e-5)
    np.testing.assert_allclose(extras["render_img"].cpu().numpy(), img * alpha, atol=2e-5)
    # culled tets keep zero cell values, visible ones get the model's
    vis = ref["project"]["tiles_touched"] > 0
    got_cell = extras["cell_values"].cpu().numpy()
    np.testing.assert_array_equal(got_cell[vis], cell[vis])
    assert not got_cell[~vis].any()
    err_ref, cnt_ref = oracle.tet_err(ref["sorted_idx"], ref["tile_ranges"], tets, pts, cell, tcam_np,
                                      extras["pixel_err"].cpu().numpy(), extras["ssim_err"].cpu().numpy())
    got = tet_err.cpu().numpy()
    scale = np.abs(err_ref).max()
    assert np.linalg.norm(got - err_ref) / np.linalg.norm(err_ref) <= 1e-3
    assert np.abs(got - err_ref).max() <= 2e-3 * scale
    cnt = extras["tet_count"].cpu().numpy()
    # hit counts: equal except for a handful of rounding-decided hits
    assert (cnt[:, 0] != cnt_ref[:, 0]).mean() < 0.01
    assert np.abs(cnt[:, 1].astype(np.int64) - cnt_ref[:, 1]).max() <= 0.02 * max(int(cnt_ref[:, 1].max()), 1) + 2
