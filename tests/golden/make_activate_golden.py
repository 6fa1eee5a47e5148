"""Generates tests/golden/activate_output.npz from the reference's own activate_output.

Run once where the reference checkout is available:
    python tests/golden/make_activate_golden.py <path-to-reference-checkout>
The reference's utils/model_util.py imports a logging helper that is not installed
here; it is replaced by an empty stand-in so the module imports.  The function
runs on CPU in float32 for SH degrees 0..3 with float32 and float16 coefficients.
"""
import os
import sys
import types

import numpy as np
import torch


def inputs(seed=7, T=500, V=300, K=15):
    g = torch.Generator().manual_seed(seed)
    vertices = torch.randn(V, 3, generator=g) * 2.0
    indices = torch.stack([torch.randperm(V, generator=g)[:4] for _ in range(T)]).int()
    circumcenters = vertices[indices.long()].mean(1) + 0.3 * torch.randn(T, 3, generator=g)
    circumcenters[5] = vertices[indices[5, 0].long()]          # zero radius: the safe_div guard
    density = torch.rand(T, 1, generator=g) * 5.0
    rgb = torch.rand(T, 3, generator=g) * 1.4 - 0.2            # some negative channels
    rgb[9] = torch.tensor([3.0, 2.5, 4.0])                     # softplus linear branch
    grd = torch.randn(T, 3, generator=g) * 0.5
    sh = torch.randn(T, K, 3, generator=g) * 0.2
    cam = torch.tensor([0.3, -4.0, 1.2])
    return dict(camera_center=cam, density=density, rgb=rgb, grd=grd, sh=sh, indices=indices,
                circumcenters=circumcenters, vertices=vertices)


def main(ref_root):
    stub = types.ModuleType("icecream")
    stub.ic = lambda *a, **k: None
    sys.modules["icecream"] = stub
    sys.path.insert(0, ref_root)
    from utils.model_util import activate_output

    x = inputs()
    out = {k: v.numpy() for k, v in x.items()}
    for deg in range(4):
        for half in (False, True):
            sh = x["sh"].half() if half else x["sh"]
            with torch.no_grad():
                f = activate_output(x["camera_center"], x["density"], x["rgb"], x["grd"], sh, x["indices"].long(),
                                    x["circumcenters"], x["vertices"], deg, 3)
            out[f"features_deg{deg}_{'f16' if half else 'f32'}"] = f.numpy()
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "activate_output.npz"), **out)


if __name__ == "__main__":
    main(sys.argv[1])
