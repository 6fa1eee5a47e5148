"""The C-ABI library loads and exports every symbol include/rm_b200.h declares
(no compute calls: there is no GPU on the CPU test box)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "rm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rm_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_exported(cuda_lib):
    from radiance_meshes_b200 import _lib
    declared = _declared_symbols()
    assert declared, "no declarations found"
    assert sorted(_lib.SYMBOLS) == declared
    for name in declared:
        assert hasattr(cuda_lib, name)
    assert cuda_lib.rm_version() >= 100
    assert cuda_lib.rm_strerror(0) == b"ok"
    assert cuda_lib.rm_bin_workspace_bytes(1000, 64) > 0


def test_struct_layout_matches_header():
    import ctypes as C
    from radiance_meshes_b200 import _lib
    assert C.sizeof(_lib.RmBinInfo) == 24
    assert C.sizeof(_lib.RmCamera) == 4 * 8 + 12 * 4
    assert _lib.RM_RECORD_FLOATS == 36 and _lib.RM_GRAD_RECORD_FLOATS == 24


def test_host_path_rejects_cpu_tensors():
    import pytest
    import torch
    from radiance_meshes_b200 import raster
    with pytest.raises(RuntimeError, match="no CPU path"):
        raster.project_and_bin(torch.zeros((1, 4), dtype=torch.int32), torch.zeros((4, 3)), {})


def test_render_grid_and_util():
    import torch
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from delaunay_rasterization.internal.util import recombine_tensors, split_tensors
    g = RenderGrid(1080, 1920, tile_width=4, tile_height=4)
    assert (g.grid_height, g.grid_width) == (270, 480)
    g = RenderGrid(17, 33, tile_width=16, tile_height=8)
    assert (g.grid_height, g.grid_width) == (3, 3)
    d = dict(a=torch.ones(2), b=3, c=torch.zeros(1), min_t=0.1)
    plain, tensors = split_tensors(d)
    assert len(tensors) == 2 and plain["b"] == 3
    back = recombine_tensors(plain, tensors)
    assert set(back) == set(d) and back["a"] is d["a"]


def test_bad_camera_is_rejected_before_any_launch(cuda_lib):
    """Host-side argument checks run before anything touches a device: a camera with NULL arrays, or
    a tile grid that does not match the image, returns RM_ERR_INVALID_ARG from every entry point that
    takes a camera (checked here where it matters most, the entry point with library-owned scratch)."""
    import ctypes as C
    from radiance_meshes_b200 import _lib
    fake = C.c_void_p(0x1000)  # never dereferenced: the call must fail first
    hits = C.byref(_lib.RmHitList(fake, fake, fake, fake))

    def call(cam, n_tets=8):
        return cuda_lib.rm_backward_static_scratch(fake, fake, fake, C.byref(cam), fake, fake, fake, fake, hits, fake,
                                                   fake, fake, fake, fake, n_tets, 4, fake, fake, None)

    cam = _lib.RmCamera()
    cam.image_height = cam.image_width = 16
    cam.tile_height = cam.tile_width = 4
    cam.grid_height = cam.grid_width = 4
    cam.tile_row_end = 4
    assert call(cam) == _lib.RM_ERR_INVALID_ARG  # the four device arrays are NULL
    cam.world_view_transform = cam.K = cam.cam_pos = cam.distortion_params = 0x1000
    cam.grid_width = 5  # does not match ceil(16 / 4)
    assert call(cam) == _lib.RM_ERR_INVALID_ARG
    cam.grid_width = 4
    cam.tile_row_end = 5  # band outside the grid
    assert call(cam) == _lib.RM_ERR_INVALID_ARG
    cam.tile_row_end = 4
    assert call(cam, n_tets=_lib.RM_STATIC_SCRATCH_MAX_TETS + 1) == _lib.RM_ERR_STATIC_SCRATCH
    assert cuda_lib.rm_launch_count() >= 0


def test_multimem_sum_rejects_bad_ranges_before_any_launch(cuda_lib):
    """rm_multimem_sum checks its arguments on the host: NULL or misaligned address, a range that is not a
    multiple of 4 floats, a rank outside the group.  An empty range is a no-op.  Nothing is launched."""
    import ctypes as C
    from radiance_meshes_b200 import _lib
    fake = C.c_void_p(0x10000)  # never dereferenced
    call = cuda_lib.rm_multimem_sum
    assert call(None, 0, 16, 0, 2, None) == _lib.RM_ERR_INVALID_ARG
    assert call(fake, 2, 16, 0, 2, None) == _lib.RM_ERR_INVALID_ARG
    assert call(fake, 0, 18, 0, 2, None) == _lib.RM_ERR_INVALID_ARG
    assert call(fake, 16, 0, 0, 2, None) == _lib.RM_ERR_INVALID_ARG
    assert call(fake, 0, 16, 2, 2, None) == _lib.RM_ERR_INVALID_ARG
    assert call(fake, 0, 16, 0, 0, None) == _lib.RM_ERR_INVALID_ARG
    assert call(C.c_void_p(0x10004), 0, 16, 0, 2, None) != 0
    assert call(fake, 16, 16, 1, 2, None) == 0
