"""Multi-GPU host logic: one process per GPU, torch.distributed for the plumbing.

The rasterizer shards two ways and needs no collective inside its kernels:

* view-parallel: every rank renders its own view of a replicated mesh; the two
  gradient tensors are summed over ranks afterwards (`allreduce_gradients`);
* tile-row bands: one large frame is split into contiguous bands of tile rows,
  every rank renders its band (the rasterizer clamps each tet's rectangle to the
  band, so a band's tile lists are exactly the single-GPU lists of those rows),
  and the image rows are combined (`combine_band_images`).

The reference is single-GPU (nothing under delaunay_rasterization/ or train.py
touches torch.distributed); this module has no counterpart there.
The functions take the renderer as a callable so that the same logic runs on CPU
ranks (gloo) in the tests.
"""
import numpy as np
import torch
import torch.distributed as dist


def _covering_view(grads):
    """If the tensors are contiguous views of one storage, a flat view of that storage from the first to the
    last of them (the gaps between them are padding); else None."""
    if len(grads) < 2 or any(not g.is_contiguous() or g.dtype != grads[0].dtype for g in grads):
        return None
    base = grads[0].untyped_storage().data_ptr()
    if any(g.untyped_storage().data_ptr() != base for g in grads):
        return None
    lo = min(g.storage_offset() for g in grads)
    hi = max(g.storage_offset() + g.numel() for g in grads)
    if hi - lo > 2 * sum(g.numel() for g in grads):
        return None
    return torch.empty(0, dtype=grads[0].dtype, device=grads[0].device).set_(
        grads[0].untyped_storage(), lo, (hi - lo,))


def allreduce_gradients(grads, group=None):
    """Sum each gradient tensor over the ranks, in place. Returns the list.  Tensors that share one
    allocation (as the two gradients of the rasterizer's backward pass do) are summed with one call."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        flat = _covering_view(grads)
        if flat is not None:
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        else:
            for g in grads:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
    return grads


class OverlappedGradientSum:
    """Sums the rasterizer's gradients over the ranks while its backward pass is still running.

    The backward pass finishes the cell-value gradients range by range (raster.set_gradient_sink);
    every finished range is all-reduced on a communication stream while the next range is being
    finished on the compute stream, the vertex gradients (which every range adds to) last.  After
    the backward pass returns, the compute stream has been made to wait for the last collective, so
    the gradients a caller sees are the sums.  Use as a context manager around the backward call, or
    install()/remove() around a training loop.
    """

    def __init__(self, group=None, chunks=4, device=None):
        self.group = group
        self.chunks = chunks
        self.device = device
        self.comm = None
        self.events = []   # (start, end) CUDA events of every collective, if timing is on
        self.timing = False

    def _active(self):
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    def __call__(self, t):
        if not self._active():
            return
        cur = torch.cuda.current_stream(t.device)
        if self.comm is None:
            self.comm = torch.cuda.Stream(t.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        self.comm.wait_event(ready)
        with torch.cuda.stream(self.comm):
            if self.timing:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(self.comm)
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
            if self.timing:
                b.record(self.comm)
                self.events.append((a, b))
        t.record_stream(self.comm)

    def done(self):
        if self.comm is not None:
            torch.cuda.current_stream(self.comm.device).wait_stream(self.comm)

    def install(self):
        from . import raster
        raster.set_gradient_sink(self, self.chunks)
        return self

    def remove(self):
        from . import raster
        raster.set_gradient_sink(None)

    def __enter__(self):
        return self.install()

    def __exit__(self, *exc):
        self.remove()
        return False


class MultimemGradientSum(OverlappedGradientSum):
    """OverlappedGradientSum with the sums formed by the NVSwitch instead of NCCL's all-reduce kernels.

    The backward pass writes its gradients into a symmetric-memory buffer that is bound to an NVLink
    multicast object (torch.distributed._symmetric_memory).  For every finished range this rank's kernel
    (rm_multimem_sum) pulls the sum of its 1/N slice through the switch and stores it to all GPUs; a
    one-element NCCL all-reduce in front of it is the barrier that tells every rank the others have written
    the range, and one more at the end that all slices have been stored.  The sums are then copied out of
    the buffer, which the next backward pass reuses.  prepare() is collective and must be called by every
    rank (outside the backward pass) before the first use; it returns False where multicast is missing."""

    def __init__(self, group=None, chunks=2, device=None):
        super().__init__(group, chunks, device)
        self.buf = None
        self.mc = 0
        self.token = None
        self.kernel_events = []  # (start, end) of every rm_multimem_sum launch, if timing is on
        self.unavailable = None  # after prepare() returned False: why, on this rank

    def prepare(self, n_floats, device):
        import torch.distributed._symmetric_memory as symm
        group = self.group if self.group is not None else dist.group.WORLD
        n4 = (int(n_floats) + 3) // 4 * 4
        # every rank first says whether it can allocate symmetric memory with multicast at all; the collective
        # rendezvous is entered only if all can, so a rank that cannot never leaves the others waiting in it
        buf, reason = None, None
        try:
            from torch._C._distributed_c10d import _SymmetricMemory
            if not _SymmetricMemory.has_multicast_support(torch._C._autograd.DeviceType.CUDA,
                                                          torch.device(device).index or 0):
                reason = "no multicast support on this device"
            else:
                buf = symm.empty(n4, dtype=torch.float32, device=device)
                buf.zero_()
        except Exception as e:
            buf, reason = None, f"{type(e).__name__}: {str(e)[:160]}"
        self.unavailable = reason
        flag = torch.tensor([0 if buf is None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            return False
        handle = None
        try:
            handle = symm.rendezvous(buf, group)
            if not handle.multicast_ptr:
                handle, self.unavailable = None, "rendezvous returned no multicast address"
        except Exception as e:  # e.g. the processes may not exchange memory handles in this container
            self.unavailable = f"{type(e).__name__}: {str(e)[:160]}"
        flag.fill_(0 if handle is None else 1)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            return False
        self.buf, self.mc, self._handle = buf, int(handle.multicast_ptr), handle
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        torch.cuda.synchronize(device)
        return True

    def allocate(self, n_floats, device):
        if self.buf is None or not self._active() or self.buf.numel() < n_floats or self.buf.device != device:
            return None
        return self.buf[:n_floats]

    def _owns(self, t):
        return self.buf is not None and t.device == self.buf.device and \
            0 <= t.data_ptr() - self.buf.data_ptr() <= 4 * (self.buf.numel() - t.numel())

    def __call__(self, t):
        if not self._active():
            return
        if not self._owns(t):  # gradients in ordinary memory: NCCL sums them
            return super().__call__(t)
        from . import _lib
        begin = (t.data_ptr() - self.buf.data_ptr()) // 4
        end = (begin + t.numel() + 3) // 4 * 4  # the buffer is padded with zeros to a multiple of 4 floats
        assert begin % 4 == 0
        cur = torch.cuda.current_stream(t.device)
        if self.comm is None:
            self.comm = torch.cuda.Stream(t.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        self.comm.wait_event(ready)
        with torch.cuda.stream(self.comm):
            if self.timing:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(self.comm)
            dist.all_reduce(self.token, op=dist.ReduceOp.SUM, group=self.group)  # every rank has written the range
            if self.timing:
                m = torch.cuda.Event(enable_timing=True)
                m.record(self.comm)
            _lib.check(_lib.load().rm_multimem_sum(self.mc, begin, end, self.rank, self.world,
                                                   self.comm.cuda_stream))
            if self.timing:
                b.record(self.comm)
                self.events.append((a, b))
                self.kernel_events.append((m, b))

    def done(self):
        if self.comm is not None and self.buf is not None and self._active():
            with torch.cuda.stream(self.comm):
                dist.all_reduce(self.token, op=dist.ReduceOp.SUM, group=self.group)  # every slice has been stored
        super().done()

    def export(self, flat):
        return flat.clone() if self._owns(flat) else flat


def tile_row_bands(grid_height, world_size, row_weights=None):
    """Split tile rows [0, grid_height) into world_size contiguous bands.

    row_weights[r] is the work of tile row r (e.g. its number of (tile, tet)
    pairs); bands are cut where the running weight crosses k/world_size of the
    total, so every rank computes the same cuts from the same weights without
    communicating. Without weights the rows are split evenly. Bands may be empty
    when there are more ranks than rows.
    """
    if row_weights is None:
        w = np.ones(grid_height, np.float64)
    else:
        w = np.asarray(row_weights, np.float64).reshape(-1)
        assert w.shape[0] == grid_height
        if w.sum() <= 0:
            w = np.ones(grid_height, np.float64)
    cum = np.concatenate([[0.0], np.cumsum(w)])
    cuts = [0]
    for k in range(1, world_size):
        target = cum[-1] * k / world_size
        r = int(np.searchsorted(cum, target, side="left"))
        cuts.append(min(max(r, cuts[-1]), grid_height))
    cuts.append(grid_height)
    return [(cuts[k], cuts[k + 1]) for k in range(world_size)]


def rebalance_bands(bands, times, row_weights):
    """New bands from the measured time of the current ones (a renderer in a sequence does this between
    frames).  Rank r took times[r] for bands[r]; its time is spread over its rows in proportion to
    row_weights, and the new cuts are placed where the running time crosses k/N of the total.  Every rank
    calls this with the same (all-gathered) times and gets the same bands."""
    w = np.asarray(row_weights, np.float64).reshape(-1)
    gh = w.shape[0]
    dens = np.zeros(gh, np.float64)
    for (a, b), t in zip(bands, times):
        if b > a:
            ww = w[a:b]
            tot = ww.sum()
            dens[a:b] = float(t) * (ww / tot if tot > 0 else np.full(b - a, 1.0 / (b - a)))
    return tile_row_bands(gh, len(bands), dens)


def row_weights_from_rects(rect_tile_space, tiles_touched, grid_height):
    """Work per tile row from the per-tet rectangles: sum over tets of the rectangle
    width for every row the rectangle covers (a difference array over rows)."""
    rect = rect_tile_space.to(torch.int64)
    vis = tiles_touched > 0
    width = (rect[:, 2] - rect[:, 0]) * vis
    diff = torch.zeros(grid_height + 1, dtype=torch.int64, device=rect.device)
    diff.index_add_(0, rect[:, 1].clamp(0, grid_height), width)
    diff.index_add_(0, rect[:, 3].clamp(0, grid_height), -width)
    return torch.cumsum(diff, 0)[:grid_height]


_POP16 = {}


def pixel_hits_per_unit(hit_counts, hit_masks, tile_ranges, units_per_tile=1):
    """(pixel, entry) hits of every hit-list unit of the previous frame: the population count of the per-pixel
    bit sets the forward pass recorded (RmHitList.masks), summed per unit.  Returns int64 [G * units_per_tile]."""
    dev = hit_counts.device
    lut = _POP16.get(dev)
    if lut is None:
        lut = _POP16[dev] = torch.tensor([bin(i).count("1") for i in range(65536)], device=dev, dtype=torch.int64)
    counts = hit_counts.to(torch.int64)
    S = units_per_tile
    n_units = counts.shape[0]
    nbatch = (counts + 15) // 16
    unit = torch.arange(n_units, device=dev, dtype=torch.int64)
    start = tile_ranges[:, 0].to(torch.int64)
    length = (tile_ranges[:, 1] - tile_ranges[:, 0]).to(torch.int64)
    base = start[unit // S] * S + (unit % S) * length[unit // S] + 16 * unit  # first mask slot of the unit
    owner = torch.repeat_interleave(unit, nbatch)
    first = torch.cumsum(nbatch, 0) - nbatch
    within = torch.arange(int(nbatch.sum().item()), device=dev, dtype=torch.int64) - first[owner]
    slots = (base[owner] + 16 * within)[:, None] + torch.arange(16, device=dev, dtype=torch.int64)[None, :]
    bits = hit_masks[slots.reshape(-1)].to(torch.int64) & 0xFFFF
    per_batch = lut[bits].reshape(-1, 16).sum(1)
    out = torch.zeros(n_units, dtype=torch.int64, device=dev)
    out.index_add_(0, owner, per_batch)
    return out


def row_weights_from_walk(n_contributors, rect_tile_space, tiles_touched, grid_height, tile_height, walk_share=0.75,
                          hit_counts=None, tile_width=None, pixel_hits=None):
    """Work per tile row for balancing bands, from the previous frame of a sequence, blended from what the
    integration kernel's time follows and the row's (tile, tet) pairs (what the list build's time follows);
    `walk_share` is the integration kernel's share of a frame's time.  Every rank computes the same weights
    from the same tensors.

    The integration term per tile: with `hit_counts` (RmHitList.counts of the previous frame) and `tile_width`,
    4 * (entries examined = the longest walk among the tile's pixels) + 20 * (entries evaluated) + 5.5 *
    (pixel hits, `pixel_hits_per_unit`; 90 * entries evaluated if those are not given) - the instruction counts of the
    phases of the forward kernel; without them the sum of the pixels' walk lengths."""
    H, W = n_contributors.shape[0], n_contributors.shape[1]
    nc = n_contributors.reshape(H, W).to(torch.float64)
    pad_h = grid_height * tile_height - H
    if pad_h > 0:
        nc = torch.cat([nc, torch.zeros((pad_h, W), dtype=nc.dtype, device=nc.device)])
    if hit_counts is not None and tile_width is not None:
        grid_width = -(-W // tile_width)
        pad_w = grid_width * tile_width - W
        if pad_w > 0:
            nc = torch.cat([nc, torch.zeros((nc.shape[0], pad_w), dtype=nc.dtype, device=nc.device)], dim=1)
        examined = nc.reshape(grid_height, tile_height, grid_width, tile_width).amax(dim=(1, 3))
        evaluated = hit_counts.to(torch.float64).reshape(grid_height, grid_width, -1).sum(-1)
        if pixel_hits is not None:
            hits = pixel_hits.to(torch.float64).reshape(grid_height, grid_width, -1).sum(-1)
            walk = (4.0 * examined + 20.0 * evaluated + 5.5 * hits).sum(1)
        else:
            walk = (4.0 * examined + 90.0 * evaluated).sum(1)
    else:
        walk = nc.sum(1).reshape(grid_height, tile_height).sum(1)
    pairs = row_weights_from_rects(rect_tile_space, tiles_touched, grid_height).to(torch.float64)
    walk = walk / walk.sum().clamp_min(1.0)
    pairs = pairs / pairs.sum().clamp_min(1.0)
    return walk_share * walk + (1.0 - walk_share) * pairs


def combine_band_images(local_image, band, tile_height, group=None, bands=None):
    """Full image from per-rank band images.

    local_image is full-size [H, W, C] with valid rows only inside the rank's band
    (other rows are ignored). Returns the full image on every rank.  With `bands` (the
    bands of all ranks, as tile_row_bands returns them) only the band rows travel, in one
    all-gather of equally sized, padded blocks; without it the images are summed.
    """
    H = local_image.shape[0]
    r0, r1 = band
    y0, y1 = min(r0 * tile_height, H), min(r1 * tile_height, H)
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    if multi and bands is not None:
        rows = [(min(b0 * tile_height, H), min(b1 * tile_height, H)) for b0, b1 in bands]
        m = max(1, max(b - a for a, b in rows))
        send = torch.zeros((m,) + tuple(local_image.shape[1:]), dtype=local_image.dtype, device=local_image.device)
        send[:y1 - y0] = local_image[y0:y1]
        recv = [torch.empty_like(send) for _ in rows]
        dist.all_gather(recv, send, group=group)
        out = torch.zeros_like(local_image)
        for (a, b), block in zip(rows, recv):
            out[a:b] = block[:b - a]
        return out
    out = torch.zeros_like(local_image)
    out[y0:y1] = local_image[y0:y1]
    if multi:
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
    return out


def render_view_parallel(render_backward_fn, views, rank, world_size, group=None, zero_like=None):
    """Each rank renders views[rank::world_size] and the gradients are summed.

    render_backward_fn(view) -> (image, vertices_grad, cell_values_grad).
    Returns (list of local images, vertices_grad, cell_values_grad) with the
    gradients summed over all views of all ranks.

    With fewer views than ranks some ranks have nothing to render but still have to join the
    collective: `zero_like` = (tensor shaped like vertices_grad, tensor shaped like
    cell_values_grad) tells them what to contribute.  Without it the call raises on EVERY
    rank before any collective is entered (all ranks see the same `views`), instead of
    leaving the ranks that do have views blocked in the all-reduce.
    """
    if len(views) < world_size and zero_like is None:
        raise ValueError(f"{len(views)} view(s) for {world_size} ranks: pass zero_like=(vertices_grad-like, "
                         "cell_values_grad-like) so that ranks without a view can join the gradient sum")
    images, vg, cg = [], None, None
    for v in views[rank::world_size]:
        img, g_v, g_c = render_backward_fn(v)
        images.append(img)
        vg = g_v.clone() if vg is None else vg + g_v
        cg = g_c.clone() if cg is None else cg + g_c
    if vg is None:
        vg, cg = torch.zeros_like(zero_like[0]), torch.zeros_like(zero_like[1])
    allreduce_gradients([vg, cg], group)
    return images, vg, cg


def render_band_split(render_band_fn, grid_height, tile_height, rank, world_size, row_weights=None, group=None,
                      bands=None):
    """One frame split over the ranks by tile-row bands.

    render_band_fn((row_begin, row_end)) -> full-size image whose band rows are valid.
    `bands`: the bands to use (e.g. from rebalance_bands); else they are cut from row_weights.
    Returns (full image on every rank, this rank's band).
    """
    if bands is None:
        bands = tile_row_bands(grid_height, world_size, row_weights)
    band = bands[rank]
    if band[1] > band[0]:
        local = render_band_fn(band)
    else:
        local = None
    if local is None:
        # a rank without rows still has to join the collective with the right shape
        local = render_band_fn((0, 0))
    return combine_band_images(local, band, tile_height, group, bands=bands), band
