"""Fused feature activation for the no-grad rendering path.

`activate_output` has the signature of the reference's function of the same name
(utils/model_util.py:93-105): per-tet density, base colour, colour gradient and
spherical-harmonics coefficients in, the [T,7] cell values the rasterizer
consumes out.  One CUDA kernel instead of about twenty torch kernels; forward
only (the reference's rendering/benchmark callers run it under torch.no_grad()).
"""
import ctypes as C

import torch

from . import _lib
from .raster import _ptr, _require_cuda, _stream


def activate_output(camera_center, density, rgb, grd, sh, indices, circumcenters, vertices, current_sh_deg,
                    max_sh_deg):
    _require_cuda(vertices, "vertices")
    if torch.is_grad_enabled() and any(t.requires_grad for t in (density, rgb, grd, sh, vertices)):
        raise RuntimeError("rm_b200 activate_output is forward-only: call it under torch.no_grad()")
    lib = _lib.load()
    dev = vertices.device
    T = indices.shape[0]
    f32 = lambda t: t.detach().to(device=dev, dtype=torch.float32).contiguous()
    cam = f32(camera_center).reshape(-1)
    dens = f32(density).reshape(-1)
    rgb_, grd_ = f32(rgb).reshape(-1, 3), f32(grd).reshape(-1, 3)
    cc, verts = f32(circumcenters).reshape(-1, 3), f32(vertices)
    idx = indices.contiguous().to(torch.int32)
    sh_ = sh.detach().to(dev)
    if sh_.dtype not in (torch.float16, torch.float32):
        sh_ = sh_.float()
    sh_ = sh_.reshape(T, sh_.numel() // (3 * T) if T else 0, 3).contiguous()
    assert dens.shape[0] == T and rgb_.shape[0] == T and grd_.shape[0] == T and cc.shape[0] == T
    with torch.cuda.device(dev):
        features = torch.empty((T, 7), dtype=torch.float32, device=dev)
        _lib.check(lib.rm_activate_output(_ptr(cam), _ptr(dens), _ptr(rgb_), _ptr(grd_), _ptr(sh_),
                                          int(sh_.dtype == torch.float16), _ptr(idx), _ptr(cc), _ptr(verts), T,
                                          int(current_sh_deg), int(sh_.shape[1]), _ptr(features), _stream(dev)))
    return features
