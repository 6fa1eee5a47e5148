"""Generates tests/golden/camera_dicts.npz from the reference's own camera class.

    python tests/golden/make_camera_golden.py <path-to-reference-checkout>

For a handful of poses it builds data/camera.py `Camera(colmap_id, R, T, fovx, fovy, image,
data_device="cpu")` the way utils/compare_quad.py:59-100 does (R = viewmat[:3,:3].T,
T = viewmat[:3,3]) and stores what `Camera.to_dict("cpu")` (data/camera.py:72-91) returns:
`world_view_transform`, `cam_pos`, `K`, `fovx`, `fovy`, `distortion_params`, `camera_type`,
plus the inputs (view matrix, image size, field of view).  The tests check that
radiance_meshes_b200.scenes.make_tcam, fed the same pose, produces the same dictionary, so the
camera convention every parity test and the bench use is the reference's.  The absent
`icecream` helper is replaced by an empty stand-in; nothing else of the reference is touched.
"""
import math
import os
import sys
import types

import numpy as np
import torch


def poses():
    """(name, eye, target, up, height, width, vertical fov in degrees)."""
    out = [("config1", (0.0, 0.0, 3.0), (0.0, 0.0, 0.0), (0.0, 1.0, 0.0), 128, 128, 60.0)]
    for k in (0, 1, 3, 6):
        ang = 2 * math.pi * k / 8
        out.append((f"ring{k}", (3.0 * math.cos(ang), 0.0, 3.0 * math.sin(ang)), (0.0, 0.0, 0.0), (0.0, 1.0, 0.0),
                    1080, 1920, 60.0))
    out.append(("oblique", (1.3, -0.7, 2.1), (0.2, 0.1, -0.3), (0.1, 1.0, 0.2), 270, 480, 75.0))
    return out


def main(ref_root):
    stub = types.ModuleType("icecream")
    stub.ic = lambda *a, **k: None
    sys.modules["icecream"] = stub
    sys.path.insert(0, ref_root)
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.dirname(os.path.dirname(here)))
    from data.camera import Camera  # the reference's class
    from radiance_meshes_b200 import scenes

    store = {}
    names = []
    for name, eye, target, up, H, W, fov in poses():
        viewmat = scenes.look_at(eye, target, up)  # world -> camera, 4x4, float64
        fovy = math.radians(fov)
        fy = H / (2 * math.tan(fovy / 2))
        fovx = 2 * math.atan(W / (2 * fy))
        cam = Camera(colmap_id=0, R=viewmat[:3, :3].T.copy(), T=viewmat[:3, 3].copy(), fovx=fovx, fovy=fovy,
                     image=torch.zeros((3, H, W)), data_device="cpu")
        d = cam.to_dict("cpu")
        names.append(name)
        store[f"{name}/viewmat"] = viewmat
        store[f"{name}/size_fov"] = np.array([H, W, fov], np.float64)
        for key in ("world_view_transform", "cam_pos", "K", "distortion_params"):
            store[f"{name}/{key}"] = d[key].numpy()
        store[f"{name}/scalars"] = np.array([d["image_height"], d["image_width"], d["fovy"], d["fovx"],
                                             d["camera_type"]], np.float64)
    store["names"] = np.array(names)
    np.savez_compressed(os.path.join(here, "camera_dicts.npz"), **store)
    print("wrote", len(names), "poses")


if __name__ == "__main__":
    main(sys.argv[1])
