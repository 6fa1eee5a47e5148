"""rm_backward_static_scratch: the backward pass for hosts that cannot allocate
device memory when it runs (an engine plugin working on buffers it was handed, a
fixed memory budget, a callback where cudaMalloc is off limits).  Its scratch is
a static device array inside the library, so the call takes inputs and outputs
only.

Checked here, through the C ABI: two calls in a row (different upstream
gradients, so stale sums left in the shared array would show) give the same
vertex and cell-value gradients as rm_backward with a caller-provided scratch,
and a mesh larger than the array is refused with a clear error.
Collected last on purpose: a failure here cannot hide any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import scene_util

pytestmark = pytest.mark.gpu

GRAD_TOL = 1e-3


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_static_scratch_backward_matches_rm_backward(cuda_lib):
    from radiance_meshes_b200 import _lib, raster
    from radiance_meshes_b200.render import tcam_to_device
    dev = torch.device("cuda:0")
    pts, tets, cell = scene_util.small_scene(400, seed=31)
    H, W = 48, 64
    tcam = tcam_to_device(scene_util.camera(H=H, W=W, tile=4), dev)
    indices = torch.tensor(tets, device=dev, dtype=torch.int32)
    vertices = torch.tensor(pts, device=dev)
    cells = torch.tensor(cell, device=dev)
    jitter = torch.tensor(scene_util.jitter(H, W, 5), device=dev)
    T, V = indices.shape[0], vertices.shape[0]
    assert T <= _lib.RM_STATIC_SCRATCH_MAX_TETS

    bctx = raster.project_and_bin(indices, vertices, tcam)
    n_keys, _ = raster.read_info(bctx)
    sorted_idx = raster.build_tile_lists(bctx, n_keys)
    cam = bctx["cam"]
    records = raster.pack_records(indices, vertices, cells, cam, bctx["tiles_touched"])
    out, dist, nc, hm = raster.forward(sorted_idx, bctx["tile_ranges"], records, cam, jitter)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    gen = torch.Generator(device="cpu").manual_seed(7)
    for call in range(2):
        g_img = torch.randn((H, W, 4), generator=gen).to(dev)
        g_dist = (0.05 * torch.randn((H, W, 5), generator=gen)).to(dev)
        # existing entry point, caller-provided scratch
        scratch = torch.empty((T, _lib.RM_GRAD_RECORD_FLOATS), device=dev)
        vg_ref = torch.empty((V, 3), device=dev)
        cg_ref = torch.empty((T, 7), device=dev)
        _lib.check(cuda_lib.rm_backward(_p(sorted_idx), _p(bctx["tile_ranges"]), _p(records), cam.ref, _p(jitter),
                                        _p(out), _p(dist), _p(nc), raster.hit_list_ref(hm), _p(g_img), _p(g_dist), _p(indices), _p(vertices),
                                        _p(cells), T, V, _p(scratch), _p(vg_ref), _p(cg_ref), stream))
        # new entry point: outputs pre-filled with garbage, no scratch argument
        vg = torch.full((V, 3), 123.0, device=dev)
        cg = torch.full((T, 7), -7.0, device=dev)
        _lib.check(cuda_lib.rm_backward_static_scratch(
            _p(sorted_idx), _p(bctx["tile_ranges"]), _p(records), cam.ref, _p(jitter), _p(out), _p(dist), _p(nc),
            raster.hit_list_ref(hm), _p(g_img), _p(g_dist), _p(indices), _p(vertices), _p(cells), T, V, _p(vg), _p(cg),
            stream))
        torch.cuda.synchronize()
        assert vg_ref.abs().max() > 0 and cg_ref.abs().max() > 0
        assert _rel(vg, vg_ref) <= GRAD_TOL, f"call {call}: vertex gradients differ"
        assert _rel(cg, cg_ref) <= GRAD_TOL, f"call {call}: cell-value gradients differ"


def test_static_scratch_rejects_oversized_mesh(cuda_lib):
    from radiance_meshes_b200 import _lib
    dev = torch.device("cuda:0")
    dummy = torch.zeros(64, device=dev)
    cam = _lib.RmCamera()
    cam.image_height = cam.image_width = 16
    cam.tile_height = cam.tile_width = 4
    cam.grid_height = cam.grid_width = 4
    cam.tile_row_end = 4
    rc = cuda_lib.rm_backward_static_scratch(
        _p(dummy), _p(dummy), _p(dummy), C.byref(cam), _p(dummy), _p(dummy), _p(dummy), _p(dummy),
        C.byref(_lib.RmHitList(_p(dummy), _p(dummy), _p(dummy), _p(dummy))),
        _p(dummy), _p(dummy), _p(dummy), _p(dummy), _p(dummy), _lib.RM_STATIC_SCRATCH_MAX_TETS + 1, 4, _p(dummy),
        _p(dummy), None)
    assert rc == _lib.RM_ERR_STATIC_SCRATCH
    assert b"RM_STATIC_SCRATCH_MAX_TETS" in cuda_lib.rm_strerror(rc)
