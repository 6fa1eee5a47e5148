"""activate_output on the GPU against the reference fixture and the numpy oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import activate_oracle as ao

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "activate_output.npz")
TOL = 5e-6   # float32; the kernel and torch differ only in summation order and exp/log1p rounding


def _run(g, sh, deg):
    from radiance_meshes_b200.activate import activate_output
    dev = torch.device("cuda:0")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    with torch.no_grad():
        out = activate_output(t(g["camera_center"]), t(g["density"]), t(g["rgb"]), t(g["grd"]), t(sh),
                              t(g["indices"]), t(g["circumcenters"]), t(g["vertices"]), deg, 3)
    return out.cpu().numpy()


@pytest.mark.parametrize("deg", [0, 1, 2, 3])
@pytest.mark.parametrize("half", [False, True])
def test_matches_reference_fixture(deg, half):
    g = np.load(GOLDEN)
    sh = g["sh"].astype(np.float16) if half else g["sh"]
    got = _run(g, sh, deg)
    want = g[f"features_deg{deg}_{'f16' if half else 'f32'}"]
    np.testing.assert_array_equal(got[:, 0], want[:, 0])
    np.testing.assert_allclose(got, want, rtol=TOL, atol=TOL)
    assert np.all(got[5, 4:] == 0)


def test_large_random_against_oracle_deg4():
    rng = np.random.default_rng(3)
    T, V, K = 200_000, 50_000, 24
    g = dict(vertices=rng.normal(size=(V, 3)).astype(np.float32) * 3,
             indices=rng.integers(0, V, size=(T, 4)).astype(np.int32),
             density=rng.random((T, 1), dtype=np.float32) * 4, rgb=rng.random((T, 3), dtype=np.float32),
             grd=rng.normal(size=(T, 3)).astype(np.float32), camera_center=np.array([1, 2, -7], np.float32))
    g["circumcenters"] = (g["vertices"][g["indices"]].mean(1) + rng.normal(size=(T, 3)) * 0.5).astype(np.float32)
    sh = (rng.normal(size=(T, K, 3)) * 0.1).astype(np.float16)
    got = _run(g, sh, 4)
    want = ao.activate_output(g["camera_center"], g["density"], g["rgb"], g["grd"], sh, g["indices"],
                              g["circumcenters"], g["vertices"], 4)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def test_empty_and_bad_arguments():
    from radiance_meshes_b200.activate import activate_output
    dev = torch.device("cuda:0")
    z = lambda *s: torch.zeros(*s, device=dev)
    out = activate_output(z(3), z(0, 1), z(0, 3), z(0, 3), z(0, 15, 3), torch.zeros(0, 4, dtype=torch.int32, device=dev),
                          z(0, 3), z(4, 3), 3, 3)
    assert out.shape == (0, 7)
    with pytest.raises(RuntimeError):   # degree 3 needs 15 coefficients, 8 given
        activate_output(z(3), z(2, 1), z(2, 3), z(2, 3), z(2, 8, 3), torch.zeros(2, 4, dtype=torch.int32, device=dev),
                        z(2, 3), z(4, 3), 3, 3)
    with pytest.raises(RuntimeError):   # forward-only
        with torch.enable_grad():
            activate_output(z(3), z(2, 1), z(2, 3).requires_grad_(), z(2, 3), z(2, 15, 3),
                            torch.zeros(2, 4, dtype=torch.int32, device=dev), z(2, 3), z(4, 3), 3, 3)
