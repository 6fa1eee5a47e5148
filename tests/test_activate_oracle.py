"""The numpy restatement of activate_output against outputs of the reference's own function."""
import os

import numpy as np
import pytest

from oracle import activate_oracle as ao

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "activate_output.npz")


@pytest.mark.parametrize("deg", [0, 1, 2, 3])
@pytest.mark.parametrize("half", [False, True])
def test_oracle_matches_reference_fixture(deg, half):
    g = np.load(GOLDEN)
    sh = g["sh"].astype(np.float16) if half else g["sh"]
    got = ao.activate_output(g["camera_center"], g["density"], g["rgb"], g["grd"], sh, g["indices"],
                             g["circumcenters"], g["vertices"], deg)
    want = g[f"features_deg{deg}_{'f16' if half else 'f32'}"]
    assert got.shape == want.shape == (len(g["indices"]), 7)
    np.testing.assert_array_equal(got[:, 0], want[:, 0])                 # density passes through
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=2e-6)          # float32 sum-order noise only
    assert np.all(got[5, 4:] == 0) and np.all(want[5, 4:] == 0)          # zero circumradius -> zero gradient


def test_safe_div_edges():
    n = np.array([1.0, -1.0, 3e38, 1.0], np.float32)
    d = np.array([0.0, 1e-39, 0.5, 2.0], np.float32)
    np.testing.assert_array_equal(ao.safe_div(n, d), np.array([0, 0, 3.40282347e38, 0.5], np.float32))
