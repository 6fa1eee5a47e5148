"""Generates tests/golden/topo_circumspheres.npz from the reference's torch geometry code.

    python tests/golden/make_topo_golden.py <path-to-reference-checkout>
For the tets of tests/golden/small_scene.npz it stores the circumcentres and radii that
utils/topo_utils.py calculate_circumcenters_torch returns in float64, the function the
reference itself uses for per-tet circumcentres (utils/model_util.py:27-32).  The tests
check the oracle's projection-stage circumcentre and its power-of-circumsphere sort depth
(|camera - centre|^2 - radius^2) against these values.
"""
import os
import sys
import types

import numpy as np
import torch


def main(ref_root):
    stub = types.ModuleType("icecream")
    stub.ic = lambda *a, **k: None
    sys.modules["icecream"] = stub
    sys.path.insert(0, ref_root)
    from utils.topo_utils import calculate_circumcenters_torch

    here = os.path.dirname(os.path.abspath(__file__))
    g = np.load(os.path.join(here, "small_scene.npz"))
    tets = torch.from_numpy(g["vertices"])[torch.from_numpy(g["indices"]).long()].double()
    cc, r = calculate_circumcenters_torch(tets)
    np.savez_compressed(os.path.join(here, "topo_circumspheres.npz"), circumcenter=cc.numpy(),
                        radius=r.reshape(-1).numpy())


if __name__ == "__main__":
    main(sys.argv[1])
