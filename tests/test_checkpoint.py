"""Frozen-model checkpoint reader: the reference's file layout, on CPU; features on the GPU."""
import json
import os

import numpy as np
import pytest
import torch

from radiance_meshes_b200 import scenes
from radiance_meshes_b200.checkpoint import FrozenScene, circumcenters_f64


def _write_reference_style_ckpt(path, seed=0, n_points=300, max_sh_deg=2):
    """A checkpoint with the keys and shapes train.py:364-368 saves for a frozen model."""
    rng = np.random.default_rng(seed)
    pts = scenes.points_uniform(n_points, seed=seed).astype(np.float32)
    tets = scenes.delaunay(pts)
    T, n_int = tets.shape[0], n_points - 20
    K = (max_sh_deg + 1) ** 2 - 1
    sd = {"interior_vertices": torch.from_numpy(pts[:n_int]), "ext_vertices": torch.from_numpy(pts[n_int:]),
          "indices": torch.from_numpy(tets.astype(np.int32)), "empty_indices": torch.empty((0, 4), dtype=torch.int32),
          "density": torch.from_numpy(rng.lognormal(0, 1, (T, 1)).astype(np.float32)),
          "rgb": torch.from_numpy(rng.uniform(0, 1, (T, 3)).astype(np.float32)),
          "gradient": torch.from_numpy(rng.normal(0, 0.3, (T, 1, 3)).astype(np.float32)),
          "sh": torch.from_numpy(rng.normal(0, 0.1, (T, K, 3)).astype(np.float16)),
          "center": torch.zeros(1, 3), "scene_scaling": torch.tensor(2.0)}
    os.makedirs(path, exist_ok=True)
    torch.save(sd, os.path.join(path, "ckpt.pth"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({"density_offset": -3.0, "max_sh_deg": max_sh_deg, "base_min_t": 0.1, "unrelated": [1, 2]}, f)
    return sd


def test_load_reference_style_checkpoint_cpu(tmp_path):
    sd = _write_reference_style_ckpt(tmp_path)
    sc = FrozenScene.load_ckpt(tmp_path, device="cpu")
    assert sc.vertices.shape[0] == sd["interior_vertices"].shape[0] + sd["ext_vertices"].shape[0]
    assert sc.indices.dtype == torch.int32 and torch.equal(sc.indices, sd["indices"])
    assert sc.sh.dtype == torch.float16 and sc.sh.shape[1] == 8
    assert sc.gradient.shape == (sd["indices"].shape[0], 3)
    assert sc.max_sh_deg == 2 and sc.density_offset == -3.0 and abs(sc.min_t - 0.2) < 1e-7
    # circumcentres: equidistant from the four vertices
    t = sc.vertices[sc.indices.long()].double()
    r = (t - sc.circumcenters.double()[:, None]).norm(dim=-1)
    assert float(((r - r[:, :1]).abs() / r[:, :1]).max()) < 1e-4
    # round trip through save_ckpt
    sc.save_ckpt(tmp_path / "again")
    sc2 = FrozenScene.load_ckpt(tmp_path / "again", device="cpu")
    for name in ("vertices", "indices", "density", "rgb", "gradient", "sh", "circumcenters"):
        assert torch.equal(getattr(sc, name), getattr(sc2, name)), name
    assert abs(sc2.min_t - sc.min_t) < 1e-7


def test_missing_keys_are_reported(tmp_path):
    _write_reference_style_ckpt(tmp_path)
    sd = torch.load(tmp_path / "ckpt.pth")
    del sd["sh"]
    torch.save(sd, tmp_path / "ckpt.pth")
    with pytest.raises(KeyError, match="sh"):
        FrozenScene.load_ckpt(tmp_path, device="cpu")


def test_circumcenters_match_reference_fixture():
    here = os.path.join(os.path.dirname(__file__), "golden")
    g, t = np.load(os.path.join(here, "small_scene.npz")), np.load(os.path.join(here, "topo_circumspheres.npz"))
    cc = circumcenters_f64(torch.from_numpy(g["vertices"]), torch.from_numpy(g["indices"]))
    err = np.abs(cc.numpy().astype(np.float64) - t["circumcenter"]).max(1) / t["radius"]
    assert err.max() < 1e-6


@pytest.mark.gpu
def test_cell_values_from_checkpoint_gpu(tmp_path):
    from oracle import activate_oracle as ao
    _write_reference_style_ckpt(tmp_path, seed=3, max_sh_deg=3)
    sc = FrozenScene.load_ckpt(tmp_path, device="cuda:0")
    cam = torch.tensor([0.5, -3.0, 1.0])
    got = sc.get_cell_values(cam).cpu().numpy()
    want = ao.activate_output(cam.numpy(), sc.density.cpu().numpy(), sc.rgb.cpu().numpy(), sc.gradient.cpu().numpy(),
                              sc.sh.cpu().numpy(), sc.indices.cpu().numpy(), sc.circumcenters.cpu().numpy(),
                              sc.vertices.cpu().numpy(), 3)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def test_ply_round_trip(tmp_path):
    """ckpt.ply with the element and property names of models/base_model.py:107-151."""
    import numpy as np
    from radiance_meshes_b200 import checkpoint
    rng = np.random.default_rng(5)
    V, T, K = 40, 57, 8
    vertices = rng.normal(size=(V, 3)).astype(np.float32)
    indices = rng.integers(0, V, (T, 4)).astype(np.int32)
    density = rng.uniform(0, 3, T).astype(np.float32)
    grd = rng.normal(size=(T, 3)).astype(np.float32)
    rgb = rng.uniform(0, 1, (T, 3)).astype(np.float32)
    sh = rng.normal(size=(T, K, 3)).astype(np.float32)
    path = tmp_path / "sub" / "ckpt.ply"
    checkpoint.write_ply(path, vertices, indices, density, grd, rgb, sh)
    head = open(path, "rb").read(1200).decode("latin1")
    assert head.startswith("ply\nformat binary_little_endian 1.0\nelement vertex 40\n")
    for name in ("element tetrahedron 57", "property list uchar int indices", "property float s",
                 "property float grd_z", "property float sh_0_r", "property float sh_8_b"):
        assert name in head
    back = checkpoint.read_ply(path)
    np.testing.assert_array_equal(back["vertices"], vertices)
    np.testing.assert_array_equal(back["indices"], indices)
    np.testing.assert_array_equal(back["density"], density)
    np.testing.assert_array_equal(back["grd"], grd)
    np.testing.assert_array_equal(back["sh_rest"], sh)
    np.testing.assert_allclose(back["rgb"], rgb, atol=1e-6)
    # degree 0 only, no tets
    checkpoint.write_ply(tmp_path / "e.ply", vertices, np.zeros((0, 4), np.int32), np.zeros(0), np.zeros((0, 3)),
                         np.zeros((0, 3)), np.zeros((0, 0, 3)))
    e = checkpoint.read_ply(tmp_path / "e.ply")
    assert e["indices"].shape == (0, 4) and e["sh_rest"].shape == (0, 0, 3)
