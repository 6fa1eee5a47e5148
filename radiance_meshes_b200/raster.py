"""Host side of the rasterizer: torch tensors in, C-ABI calls, torch tensors out.

PyTorch is used for device memory, streams and autograd plumbing only; every
computation happens in the CUDA library.
"""
import ctypes as C

import torch

from . import _lib


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _f32c(t, device):
    if not isinstance(t, torch.Tensor):
        t = torch.as_tensor(t)
    return t.to(device=device, dtype=torch.float32).contiguous()


class CameraArgs:
    """RmCamera plus the device tensors it points at (kept alive with it)."""

    def __init__(self, tcam, device, tile_rows=None):
        self.keep = [_f32c(tcam["world_view_transform"], device), _f32c(tcam["K"], device),
                     _f32c(tcam["cam_pos"], device), _f32c(tcam["distortion_params"], device)]
        assert self.keep[0].numel() == 16 and self.keep[1].numel() == 9
        assert self.keep[2].numel() == 3 and self.keep[3].numel() == 4
        c = _lib.RmCamera()
        c.world_view_transform, c.K, c.cam_pos, c.distortion_params = [t.data_ptr() for t in self.keep]
        c.image_height = int(tcam["image_height"])
        c.image_width = int(tcam["image_width"])
        c.camera_type = int(tcam["camera_type"])
        c.fovy = float(tcam["fovy"])
        c.fovx = float(tcam["fovx"])
        c.min_t = float(tcam["min_t"])
        c.tile_height = int(tcam["tile_height"])
        c.tile_width = int(tcam["tile_width"])
        c.grid_height = int(tcam["grid_height"])
        c.grid_width = int(tcam["grid_width"])
        r0, r1 = tile_rows if tile_rows is not None else tcam.get("tile_rows", (0, c.grid_height))
        c.tile_row_begin, c.tile_row_end = int(r0), int(r1)
        # a band-restricted call zero-fills the image rows outside its band unless the caller reads the band only
        self.band_rows_only = bool(tcam.get("band_rows_only", False))
        self.c = c

    @property
    def ref(self):
        return C.byref(self.c)


def _require_cuda(t, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise RuntimeError(f"{name} must be a CUDA tensor (the rasterizer has no CPU path)")


def project_and_bin(indices, vertices, tcam, tile_rows=None):
    """Stage 1 and tile populations. Returns a dict of outputs plus the binning context."""
    _require_cuda(indices, "indices")
    _require_cuda(vertices, "vertices")
    lib = _lib.load()
    dev = vertices.device
    indices = indices.contiguous()
    if indices.dtype != torch.int32:
        indices = indices.to(torch.int32)
    verts = vertices.detach().contiguous().float()
    T, V = indices.shape[0], verts.shape[0]
    cam = CameraArgs(tcam, dev, tile_rows)
    G = cam.c.grid_height * cam.c.grid_width
    with torch.cuda.device(dev):
        tiles_touched = torch.empty((T,), dtype=torch.int32, device=dev)
        rect = torch.empty((T, 4), dtype=torch.int32, device=dev)
        vs_tetra = torch.empty((T, 3), dtype=torch.float32, device=dev)
        circumcenter = torch.empty((T, 3), dtype=torch.float32, device=dev)
        tile_ranges = torch.empty((G, 2), dtype=torch.int32, device=dev)
        info = torch.empty((3,), dtype=torch.int64, device=dev)
        ws_bytes = lib.rm_bin_workspace_bytes(T, G)
        ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
        _lib.check(lib.rm_project_and_bin(_ptr(indices), T, _ptr(verts), V, cam.ref, _ptr(tiles_touched), _ptr(rect),
                                          _ptr(vs_tetra), _ptr(circumcenter), _ptr(tile_ranges), _ptr(info),
                                          _ptr(ws), ws_bytes, _stream(dev)))
    return dict(indices=indices, vertices=verts, cam=cam, tiles_touched=tiles_touched, rect=rect, vs_tetra=vs_tetra,
                circumcenter=circumcenter, tile_ranges=tile_ranges, info=info, workspace=ws, T=T, V=V, G=G)


def read_info(ctx):
    """The one host synchronisation of the binning stage: N, visible count, status."""
    host = ctx["info"].cpu()
    n_keys = int(host[0].item())
    ctx["n_region_keys"] = int(host[1].item())
    second = int(host[2].item())
    n_visible = second & 0xFFFFFFFF
    status = (second >> 32) & 0xFFFFFFFF
    if status & _lib.RM_STATUS_NAN_VERTEX:
        # same message as the reference's assert (tile_shader_slang.py:78)
        raise AssertionError("Tensor contains NaN values!")
    if status & _lib.RM_STATUS_BAD_INDEX:
        raise IndexError("rm_b200: indices name a vertex outside [0, n_vertices)")
    if status & _lib.RM_STATUS_KEY_OVERFLOW or n_keys > 2**31 - 1:
        raise RuntimeError(f"rm_b200: {n_keys} (tile, tet) pairs exceed the int32 range of the tile lists")
    return n_keys, n_visible


def build_tile_lists(ctx, n_keys):
    lib = _lib.load()
    dev = ctx["vertices"].device
    with torch.cuda.device(dev):
        sorted_idx = torch.empty((n_keys,), dtype=torch.int32, device=dev)
        if n_keys > 0:
            if "n_region_keys" not in ctx:
                raise RuntimeError("rm_b200: call read_info(ctx) before build_tile_lists")
            n_region_keys = ctx["n_region_keys"]
            gh, gw = ctx["cam"].c.grid_height, ctx["cam"].c.grid_width
            nbytes = lib.rm_list_scratch_bytes(n_region_keys, gh, gw)
            if nbytes == 0:
                raise RuntimeError("rm_b200: tile grids above 2^22 regions of 8 x 4 tiles are not supported")
            scratch = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
            _lib.check(lib.rm_build_tile_lists(_ptr(ctx["rect"]), _ptr(ctx["tile_ranges"]), ctx["T"], ctx["cam"].ref,
                                               n_keys, n_region_keys, _ptr(ctx["workspace"]), _ptr(scratch), nbytes,
                                               _ptr(sorted_idx), _stream(dev)))
    return sorted_idx


def pack_records(indices, vertices, cell_values, cam, tiles_touched=None):
    lib = _lib.load()
    dev = vertices.device
    T = indices.shape[0]
    with torch.cuda.device(dev):
        records = torch.empty((T, _lib.RM_RECORD_FLOATS), dtype=torch.float32, device=dev)
        _lib.check(lib.rm_pack_records(_ptr(indices), _ptr(vertices), _ptr(cell_values), T, vertices.shape[0],
                                       cam.ref, _ptr(tiles_touched), _ptr(records), _stream(dev)))
    return records


def hit_list_ref(hits):
    """ctypes argument for a hit list given as the (counts, ids, masks) tensors forward() returns."""
    if hits is None:
        return None
    counts, ids, masks, tet_flags = hits
    return C.byref(_lib.RmHitList(_ptr(counts), _ptr(ids), _ptr(masks), _ptr(tet_flags)))


def forward(sorted_idx, tile_ranges, records, cam, ray_jitter, want_hit_masks=True):
    """Returns (output_img, distortion_img, n_contributors, hits); hits = (counts int32 [G*S], ids int32 [N*S],
    masks int16 [N*S + 16*G*S], tet_flags uint8 [T]) are the hit lists backward() walks, None if not requested."""
    lib = _lib.load()
    dev = records.device
    H, W = cam.c.image_height, cam.c.image_width
    full = cam.c.tile_row_begin == 0 and cam.c.tile_row_end == cam.c.grid_height
    alloc = torch.empty if (full or cam.band_rows_only) else torch.zeros
    with torch.cuda.device(dev):
        output_img = alloc((H, W, 4), dtype=torch.float32, device=dev)
        distortion_img = alloc((H, W, 5), dtype=torch.float32, device=dev)
        n_contributors = alloc((H, W, 1), dtype=torch.int32, device=dev)
        hits = None
        if want_hit_masks:
            groups = (cam.c.tile_width * cam.c.tile_height + 15) // 16
            slots = max(int(sorted_idx.shape[0]) * groups, 1)
            units = cam.c.grid_height * cam.c.grid_width * groups
            hits = (alloc((units,), dtype=torch.int32, device=dev),
                    torch.empty((slots,), dtype=torch.int32, device=dev),
                    torch.empty((slots + 16 * units,), dtype=torch.int16, device=dev),
                    torch.zeros((max(int(records.shape[0]), 1),), dtype=torch.uint8, device=dev))
        if _lib.bounds_checked():
            _lib.set_extents(list=sorted_idx.shape[0], tets=records.shape[0],
                             hit_ids=hits[1].shape[0] if hits else 0, hit_masks=hits[2].shape[0] if hits else 0,
                             units=hits[0].shape[0] if hits else 0)
        _lib.check(lib.rm_forward(_ptr(sorted_idx), _ptr(tile_ranges), _ptr(records), cam.ref, _ptr(ray_jitter),
                                  _ptr(output_img), _ptr(distortion_img), _ptr(n_contributors), hit_list_ref(hits),
                                  _stream(dev)))
    return output_img, distortion_img, n_contributors, hits


# Optional consumer of finished gradients, set by a multi-GPU job (dist.OverlappedGradientSum.install): the
# backward pass then finishes the tets in `chunks` ranges and hands every finished range of cell_values_grad,
# and vertices_grad at the end, to `sink` while the next range is still being finished.
_gradient_sink = None


def set_gradient_sink(sink, chunks=4):
    """sink(tensor) is called on the backward pass's stream, in order, with views of the two gradients as
    they become final: ranges of rows of the cell-value gradients first, the vertex gradients last;
    sink.done() once at the end.  Both gradients live in one buffer (vertex gradients first, zero-padded to a
    multiple of 4 floats, then the cell-value gradients), so the views are contiguous ranges of it.  Optional methods: sink.allocate(n_floats, device) -> a float32 tensor the gradients are
    written to (or None for an ordinary allocation), sink.export(flat) -> the tensor handed to the caller
    after done().  None removes the sink."""
    global _gradient_sink
    _gradient_sink = None if sink is None else (sink, max(1, int(chunks)))


def backward(sorted_idx, tile_ranges, records, cam, ray_jitter, output_img, distortion_img, n_contributors,
             hits, grad_output_img, grad_distortion_img, indices, vertices, cell_values):
    lib = _lib.load()
    dev = records.device
    T, V = indices.shape[0], vertices.shape[0]
    with torch.cuda.device(dev):
        grad_records = torch.empty((T, _lib.RM_GRAD_RECORD_FLOATS), dtype=torch.float32, device=dev)
        # both gradients live in one allocation (the second one 16-byte aligned), so that a multi-GPU
        # job can sum them over the ranks with a single all-reduce (dist.allreduce_gradients)
        off = (3 * V + 3) // 4 * 4
        sink = _gradient_sink
        flat = None
        if sink is not None and hasattr(sink[0], "allocate"):  # a sink may want the gradients in memory of its own
            flat = sink[0].allocate(off + 7 * T, dev)
        if flat is None:
            flat = torch.empty((off + 7 * T,), dtype=torch.float32, device=dev)
        vertices_grad = flat[:3 * V].view(V, 3)
        cell_grad = flat[off:].view(T, 7)
        if off > 3 * V:
            flat[3 * V:off].zero_()
        href = hit_list_ref(hits)
        st = _stream(dev)
        if _lib.bounds_checked():
            _lib.set_extents(list=sorted_idx.shape[0], tets=T, verts=V, hit_ids=hits[1].shape[0],
                             hit_masks=hits[2].shape[0], units=hits[0].shape[0])
        _lib.check(lib.rm_backward_integrate(_ptr(tile_ranges), _ptr(records), cam.ref, _ptr(ray_jitter),
                                             _ptr(output_img), _ptr(distortion_img), href, _ptr(grad_output_img),
                                             _ptr(grad_distortion_img), T, V, _ptr(grad_records), _ptr(vertices_grad),
                                             st))
        n_chunks = sink[1] if sink is not None and T >= 4096 else 1
        step = -(-T // n_chunks)
        step = -(-step // 256) * 256  # range starts on multiples of 256 tets
        t0 = 0
        while True:
            t1 = min(t0 + step, T)
            _lib.check(lib.rm_backward_finish(_ptr(indices), _ptr(vertices), _ptr(cell_values), t0, t1, T, cam.ref,
                                              _ptr(grad_records), href, _ptr(vertices_grad), _ptr(cell_grad), st))
            if sink is not None and t1 > t0:
                sink[0](cell_grad[t0:t1])
            t0 = t1
            if t0 >= T:
                break
        if sink is not None:
            sink[0](vertices_grad)
            sink[0].done()
            if hasattr(sink[0], "export"):  # the sums leave the sink's memory before its next use
                flat = sink[0].export(flat)
                vertices_grad = flat[:3 * V].view(V, 3)
                cell_grad = flat[off:].view(T, 7)
    return vertices_grad, cell_grad


def vertex_backward(indices, vertices, cam, tiles_touched, grad_vs, grad_cc):
    lib = _lib.load()
    dev = vertices.device
    T, V = indices.shape[0], vertices.shape[0]
    with torch.cuda.device(dev):
        vertices_grad = torch.empty((V, 3), dtype=torch.float32, device=dev)
        _lib.check(lib.rm_vertex_backward(_ptr(indices), _ptr(vertices), T, V, cam.ref, _ptr(tiles_touched),
                                          _ptr(grad_vs), _ptr(grad_cc), _ptr(vertices_grad), _stream(dev)))
    return vertices_grad


def tet_err(sorted_idx, tile_ranges, records, cam, pixel_err, ssim_err, n_tets):
    """Densification statistics: (tet_err[T,16] f32, tet_count[T,2] i32)."""
    lib = _lib.load()
    dev = records.device
    with torch.cuda.device(dev):
        err = torch.empty((n_tets, 16), dtype=torch.float32, device=dev)
        cnt = torch.empty((n_tets, 2), dtype=torch.int32, device=dev)
        if _lib.bounds_checked():
            _lib.set_extents(list=sorted_idx.shape[0], tets=n_tets)
        _lib.check(lib.rm_tet_err(_ptr(sorted_idx), _ptr(tile_ranges), _ptr(records), cam.ref, _ptr(pixel_err),
                                  _ptr(ssim_err), n_tets, _ptr(err), _ptr(cnt), _stream(dev)))
    return err, cnt
