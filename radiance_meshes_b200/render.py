"""The call a user of the rasterizer makes: one frame through the drop-in
`delaunay_rasterization` entry points, in the order the reference's render glue
uses them (utils/train_util.py:14-75), for given per-tet cell values."""
import torch

from delaunay_rasterization.internal.alphablend_tiled_slang_interp import AlphaBlendTiledRender
from delaunay_rasterization.internal.render_grid import RenderGrid
from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader


def tcam_to_device(tcam, device):
    """NumPy/CPU camera dictionary -> dictionary with CUDA tensors (data/camera.py:72-91)."""
    out = {}
    for k, v in tcam.items():
        if k in ("world_view_transform", "K", "cam_pos", "distortion_params"):
            out[k] = torch.as_tensor(v, dtype=torch.float32).to(device)
        else:
            out[k] = v
    return out


def render(indices, vertices, cell_values, tcam, ray_jitter=None, before_blend=None):
    """Returns dict(render[3,H,W], alpha[H,W] (log-transmittance), distortion_loss, mask, image, distortion_img).

    `before_blend`, if given, is called after the tile lists are built and before the first kernel that
    reads `cell_values` and `ray_jitter` is launched (a pipeline waits there for their copies to land)."""
    H, W = int(tcam["image_height"]), int(tcam["image_width"])
    device = vertices.device
    if ray_jitter is None:
        ray_jitter = 0.5 * torch.ones((H, W, 2), device=device)
    grid = RenderGrid(H, W, tile_height=int(tcam["tile_height"]), tile_width=int(tcam["tile_width"]))
    sorted_tetra_idx, tile_ranges, vs_tetra, circumcenter, mask, rect = vertex_and_tile_shader(
        indices, vertices, tcam, grid)
    if before_blend is not None:
        before_blend()
    image, distortion_img, tet_alive = AlphaBlendTiledRender.apply(
        sorted_tetra_idx, tile_ranges, indices, vertices, cell_values, grid, tcam, ray_jitter)
    total_density = (distortion_img[:, :, 2] ** 2).clip(min=1e-6)
    distortion_loss = (((distortion_img[:, :, 0] - distortion_img[:, :, 1]) + distortion_img[:, :, 4])
                       / total_density).clip(min=0)
    return dict(render=image.permute(2, 0, 1)[:3], alpha=image[..., 3], distortion_loss=distortion_loss.mean(),
                mask=mask, image=image, distortion_img=distortion_img, sorted_tetra_idx=sorted_tetra_idx,
                tile_ranges=tile_ranges, vs_tetra=vs_tetra, circumcenter=circumcenter, rect=rect)


class _FrameSlot:
    """Streams and device staging buffers of one frame in flight."""

    def __init__(self, device, own_compute_stream):
        self.compute = torch.cuda.Stream(device) if own_compute_stream else None
        self.copy_in = torch.cuda.Stream(device)
        self.copy_out = torch.cuda.Stream(device)
        self.staging = {}
        self.pkg = None


class HostFramePipeline:
    """Forward + backward of frames whose inputs and results live in pinned host memory.

    The host<->device copies run on two copy streams and overlap the kernels of the same
    frame: projection and tile-list building start as soon as vertices and indices have
    arrived, while the cell values (the largest input) are still in flight; the image and
    the distortion moments go back to the host while the backward pass runs; only the two
    gradient tensors are copied after the last kernel.  Device staging buffers for the
    inputs are allocated once per frame in flight and reused.

    `step` runs one frame to completion on the caller's stream (frames_in_flight = 1).  With
    frames_in_flight = 2, `submit` / `wait` keep two independent frames in flight, each on its
    own streams, so that the copies of one frame also overlap the kernels of the other: the
    next frame's inputs arrive while this frame's backward pass runs, and this frame's
    gradients leave while the next frame is binned.  The caller provides one set of result
    buffers per frame in flight.
    """

    def __init__(self, device, frames_in_flight=1):
        self.device = torch.device(device)
        assert frames_in_flight >= 1
        self.slots = [_FrameSlot(self.device, frames_in_flight > 1) for _ in range(frames_in_flight)]
        self.submitted = 0

    @staticmethod
    def _stage(slot, name, host_tensor, device):
        buf = slot.staging.get(name)
        if buf is None or buf.shape != host_tensor.shape or buf.dtype != host_tensor.dtype:
            buf = torch.empty(host_tensor.shape, dtype=host_tensor.dtype, device=device)
            slot.staging[name] = buf
        buf.copy_(host_tensor, non_blocking=True)
        return buf

    def submit(self, host_in, host_out, tcam, reduce_gradients=None):
        """Enqueues one frame and returns a ticket for `wait`.  host_in: indices, vertices, cell, jitter, g_img,
        g_dist (pinned).  host_out: image, dist, vg, cg (pinned; valid after `wait`).
        `reduce_gradients([vertices_grad, cell_grad])`, if given, runs after the backward pass and before the
        gradients are copied out (the sum over ranks of a multi-GPU job).  The call returns after the frame's
        one host synchronisation (the number of list entries), with the rest of the frame enqueued."""
        ticket = self.submitted
        slot = self.slots[ticket % len(self.slots)]
        self.submitted += 1
        slot.copy_out.synchronize()  # the slot's previous frame has left: its buffers are free
        cur = slot.compute if slot.compute is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.stream(cur):
            slot.pkg = self._enqueue(slot, cur, host_in, host_out, tcam, reduce_gradients)
        return ticket

    def wait(self, ticket):
        """Blocks until the frame of `ticket` is complete and its results are in host memory."""
        slot = self.slots[ticket % len(self.slots)]
        slot.copy_out.synchronize()
        return slot.pkg

    def step(self, host_in, host_out, tcam, reduce_gradients=None):
        """One frame, start to finish.  Returns the render package of the frame."""
        return self.wait(self.submit(host_in, host_out, tcam, reduce_gradients))

    def _enqueue(self, slot, cur, host_in, host_out, tcam, reduce_gradients):
        dev = self.device
        ev_geometry, ev_cells, ev_grads = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
        slot.copy_in.wait_stream(cur)  # the previous frame's kernels are done with the staging buffers
        with torch.cuda.stream(slot.copy_in):
            vertices = self._stage(slot, "vertices", host_in["vertices"], dev)
            indices = self._stage(slot, "indices", host_in["indices"], dev)
            ev_geometry.record(slot.copy_in)
            cell = self._stage(slot, "cell", host_in["cell"], dev)
            jitter = self._stage(slot, "jitter", host_in["jitter"], dev)
            ev_cells.record(slot.copy_in)
            g_img = self._stage(slot, "g_img", host_in["g_img"], dev)
            g_dist = self._stage(slot, "g_dist", host_in["g_dist"], dev)
            ev_grads.record(slot.copy_in)
        v = vertices.detach().requires_grad_(True)
        c = cell.detach().requires_grad_(True)
        cur.wait_event(ev_geometry)
        pkg = render(indices, v, c, tcam, jitter, before_blend=lambda: cur.wait_event(ev_cells))
        image, dimg = pkg["image"].detach(), pkg["distortion_img"].detach()
        slot.copy_out.wait_stream(cur)
        with torch.cuda.stream(slot.copy_out):
            host_out["image"].copy_(image, non_blocking=True)
            host_out["dist"].copy_(dimg, non_blocking=True)
        image.record_stream(slot.copy_out)
        dimg.record_stream(slot.copy_out)
        cur.wait_event(ev_grads)
        torch.autograd.backward([pkg["image"], pkg["distortion_img"]], [g_img, g_dist])
        if reduce_gradients is not None:
            reduce_gradients([v.grad, c.grad])
        slot.copy_out.wait_stream(cur)
        with torch.cuda.stream(slot.copy_out):
            host_out["vg"].copy_(v.grad, non_blocking=True)
            host_out["cg"].copy_(c.grad, non_blocking=True)
        v.grad.record_stream(slot.copy_out)
        c.grad.record_stream(slot.copy_out)
        return pkg
