"""ctypes binding of librm_b200.so (the C ABI declared in include/rm_b200.h).

There is no CPU fallback: if the library is missing, loading raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# RM_B200_LIBRARY selects another build of the same library (the tests load the bounds-checked one)
LIB_PATH = os.environ.get("RM_B200_LIBRARY") or os.path.join(_HERE, "librm_b200.so")

RM_RECORD_FLOATS = 36
RM_GRAD_RECORD_FLOATS = 24
RM_STATUS_NAN_VERTEX = 1
RM_STATUS_KEY_OVERFLOW = 2
RM_STATUS_BAD_INDEX = 4

# every symbol include/rm_b200.h declares
SYMBOLS = ["rm_strerror", "rm_version", "rm_bin_workspace_bytes", "rm_list_scratch_bytes", "rm_project_and_bin", "rm_build_tile_lists",
           "rm_pack_records", "rm_forward", "rm_backward", "rm_vertex_backward", "rm_profile_enable",
           "rm_profile_read", "rm_backward_static_scratch", "rm_tet_err",
           "rm_activate_output", "rm_forward_constant_color", "rm_launch_count",
           "rm_backward_integrate", "rm_backward_finish", "rm_debug_bounds_checked", "rm_debug_set_extent",
           "rm_debug_bounds_status", "rm_backward_constant_color", "rm_multimem_sum"]
RM_STATIC_SCRATCH_MAX_TETS = 131072
RM_ERR_STATIC_SCRATCH = -5
RM_ERR_INVALID_ARG = -1


class RmCamera(C.Structure):
    _fields_ = [("world_view_transform", C.c_void_p), ("K", C.c_void_p), ("cam_pos", C.c_void_p),
                ("distortion_params", C.c_void_p), ("image_height", C.c_int32), ("image_width", C.c_int32),
                ("camera_type", C.c_int32), ("fovy", C.c_float), ("fovx", C.c_float), ("min_t", C.c_float),
                ("tile_height", C.c_int32), ("tile_width", C.c_int32), ("grid_height", C.c_int32),
                ("grid_width", C.c_int32), ("tile_row_begin", C.c_int32), ("tile_row_end", C.c_int32)]


class RmHitList(C.Structure):
    _fields_ = [("counts", C.c_void_p), ("ids", C.c_void_p), ("masks", C.c_void_p), ("tet_flags", C.c_void_p)]


class RmBinInfo(C.Structure):
    _fields_ = [("n_keys", C.c_int64), ("n_region_keys", C.c_int64), ("n_visible", C.c_int32),
                ("status", C.c_uint32)]


_lib = None


def load():
    """Load the CUDA library, building nothing: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m radiance_meshes_b200.csrc.build` "
            "(there is no CPU fallback for the rasterizer)")
    lib = C.CDLL(LIB_PATH)
    vp, i64, sz = C.c_void_p, C.c_int64, C.c_size_t
    cam = C.POINTER(RmCamera)
    lib.rm_strerror.restype = C.c_char_p
    lib.rm_strerror.argtypes = [C.c_int]
    lib.rm_version.restype = C.c_int
    lib.rm_bin_workspace_bytes.restype = sz
    lib.rm_bin_workspace_bytes.argtypes = [i64, i64]
    lib.rm_project_and_bin.argtypes = [vp, i64, vp, i64, cam, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.rm_list_scratch_bytes.restype = sz
    lib.rm_list_scratch_bytes.argtypes = [i64, C.c_int, C.c_int]
    lib.rm_build_tile_lists.argtypes = [vp, vp, i64, cam, i64, i64, vp, vp, sz, vp, vp]
    lib.rm_pack_records.argtypes = [vp, vp, vp, i64, i64, cam, vp, vp, vp]
    hits = C.POINTER(RmHitList)
    lib.rm_forward.argtypes = [vp, vp, vp, cam, vp, vp, vp, vp, hits, vp]
    lib.rm_backward.argtypes = [vp, vp, vp, cam, vp, vp, vp, vp, hits, vp, vp, vp, vp, vp, i64, i64, vp, vp, vp, vp]
    lib.rm_backward_integrate.argtypes = [vp, vp, cam, vp, vp, vp, hits, vp, vp, i64, i64, vp, vp, vp]
    lib.rm_backward_finish.argtypes = [vp, vp, vp, i64, i64, i64, cam, vp, hits, vp, vp, vp]
    lib.rm_vertex_backward.argtypes = [vp, vp, i64, i64, cam, vp, vp, vp, vp, vp]
    lib.rm_backward_static_scratch.argtypes = [vp, vp, vp, cam, vp, vp, vp, vp, hits, vp, vp, vp, vp, vp, i64, i64, vp, vp,
                                               vp]
    lib.rm_tet_err.argtypes = [vp, vp, vp, cam, vp, vp, i64, vp, vp, vp]
    lib.rm_activate_output.argtypes = [vp, vp, vp, vp, vp, C.c_int, vp, vp, vp, i64, C.c_int, C.c_int, vp, vp]
    lib.rm_multimem_sum.argtypes = [vp, i64, i64, C.c_int, C.c_int, vp]
    lib.rm_forward_constant_color.argtypes = [vp, vp, vp, cam, C.c_float, C.c_float, vp, vp, vp, vp]
    lib.rm_backward_constant_color.argtypes = [vp, vp, vp, cam, C.c_float, C.c_float, vp, vp, vp, vp, vp, vp, vp, vp,
                                               i64, i64, vp, vp, vp, vp, vp]
    lib.rm_profile_enable.restype = None
    lib.rm_profile_enable.argtypes = [C.c_int]
    lib.rm_profile_read.argtypes = [C.c_char_p, sz, C.POINTER(C.c_float), C.c_int]
    lib.rm_launch_count.restype = C.c_int64
    lib.rm_debug_set_extent.restype = None
    lib.rm_debug_set_extent.argtypes = [C.c_int, i64]
    lib.rm_debug_bounds_status.restype = C.c_uint32
    for name in SYMBOLS:
        getattr(lib, name)
    _lib = lib
    return lib


def check(rc):
    if rc != 0:
        raise RuntimeError(f"rm_b200: {load().rm_strerror(rc).decode()} (code {rc})")


_checked = None


def bounds_checked():
    """True if the loaded library is the bounds-checked build."""
    global _checked
    if _checked is None:
        _checked = bool(load().rm_debug_bounds_checked())
    return _checked


def set_extents(**extents):
    """Bounds-checked build only: extents of caller-owned arrays (list, tets, verts, hit_ids, hit_masks, units)."""
    order = ("list", "tets", "verts", "hit_ids", "hit_masks", "units")
    lib = load()
    for k, v in extents.items():
        lib.rm_debug_set_extent(order.index(k), int(v))


def bounds_status():
    return int(load().rm_debug_bounds_status())


def launch_count():
    """Kernels this library has launched in this process so far."""
    return int(load().rm_launch_count())


def profile_enable(on=True):
    load().rm_profile_enable(1 if on else 0)


def profile_read(max_records=4096):
    """Returns [(kernel name, milliseconds)] recorded since the last read."""
    lib = load()
    names = C.create_string_buffer(64 * max_records)
    ms = (C.c_float * max_records)()
    n = lib.rm_profile_read(names, len(names), ms, max_records)
    labels = names.value.decode().split("\n")[:n]
    return list(zip(labels, [ms[i] for i in range(n)]))
