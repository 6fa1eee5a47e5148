"""Multi-rank host logic on CPU ranks (gloo, world_size 2): gradient all-reduce
for view-parallel rendering and tile-row band splitting of one frame.  The CPU
oracle stands in for the renderer, so these run without a GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import scene_util
from radiance_meshes_b200 import dist as rmdist
from radiance_meshes_b200 import scenes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _scene():
    pts, tets, cell = scene_util.small_scene(150, seed=17)
    return pts, tets, cell


def _view(k, H=32, W=40):
    return scenes.ring_camera(k, 4, H, W, 60.0, radius=2.6, tile=4, min_t=0.1)


def _oracle_render_backward(O, pts, tets, cell, tcam, rows=None):
    H, W = tcam["image_height"], tcam["image_width"]
    jit = np.full((H, W, 2), 0.5, np.float32)
    pr = O.project(tets, pts, tcam)
    tt, rect = pr["tiles_touched"], pr["rect"]
    if rows is not None:
        tt, rect = O.restrict_to_tile_rows(tt, rect, rows[0], rows[1])
    idx, ranges = O.build_lists(tt, rect, pr["vs_tetra"], tcam["grid_height"], tcam["grid_width"])
    prow = None if rows is None else (rows[0] * tcam["tile_height"], min(rows[1] * tcam["tile_height"], H))
    if prow is not None and prow[1] <= prow[0]:
        return np.zeros((H, W, 4), np.float32), None, None, idx, ranges
    out, dist_img, nc = O.forward(idx, ranges, tets, pts, cell, tcam, jit, rows=prow)
    g_img = np.ones((H, W, 4), np.float32)
    vg, cg = O.backward(idx, ranges, tets, pts, cell, tcam, jit, out, dist_img, nc, g_img,
                        np.zeros((H, W, 5), np.float32), rows=prow)
    return out, vg, cg, idx, ranges


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        pts, tets, cell = _scene()
        # --- view-parallel: 4 views over 2 ranks, gradients summed
        def rb(view):
            out, vg, cg, _, _ = _oracle_render_backward(O, pts, tets, cell, _view(view))
            return torch.from_numpy(out), torch.from_numpy(vg), torch.from_numpy(cg)
        images, vg, cg = rmdist.render_view_parallel(rb, [0, 1, 2, 3], rank, world)
        # --- fewer views than ranks: rank 1 has nothing to render and contributes zeros of the right shape;
        # without the shapes every rank raises before any collective
        one_img, vg1, cg1 = rmdist.render_view_parallel(rb, [2], rank, world, zero_like=(vg, cg))
        try:
            rmdist.render_view_parallel(rb, [2], rank, world)
            raised = False
        except ValueError:
            raised = True
        # --- band split of view 0
        tcam = _view(0)
        pr = O.project(tets, pts, tcam)
        weights = rmdist.row_weights_from_rects(torch.from_numpy(pr["rect"]), torch.from_numpy(pr["tiles_touched"]),
                                                tcam["grid_height"])
        def band_fn(band):
            out, _, _, _, _ = _oracle_render_backward(O, pts, tets, cell, tcam, rows=band)
            return torch.from_numpy(out)
        full, band = rmdist.render_band_split(band_fn, tcam["grid_height"], tcam["tile_height"], rank, world,
                                              row_weights=weights.numpy())
        # --- gradients that share one allocation are summed with a single collective, padding included
        flat = torch.arange(20, dtype=torch.float32) * (rank + 1)
        a, b = flat[:6].view(2, 3), flat[8:15].view(1, 7)
        separate = [torch.full((3,), float(rank + 1)), torch.full((2, 2), 10.0 * (rank + 1))]
        rmdist.allreduce_gradients([a, b])
        rmdist.allreduce_gradients(separate)
        # --- the switch-side gradient sum needs CUDA symmetric memory with multicast: on these CPU ranks every
        # rank learns that together (no rank is left waiting in the rendezvous) and the NCCL-style class is used
        mm = rmdist.MultimemGradientSum(chunks=2)
        mm_ok = mm.prepare(64, torch.device("cpu"))
        mm_alloc = mm.allocate(64, torch.device("cpu"))
        results[rank] = dict(mm_ok=mm_ok, mm_reason=mm.unavailable, mm_alloc_none=mm_alloc is None,
                             vg=vg.numpy(), cg=cg.numpy(), n_images=len(images), full=full.numpy(), band=band,
                             vg1=vg1.numpy(), cg1=cg1.numpy(), n_images1=len(one_img), raised=raised,
                             weights=weights.numpy(), flat=flat.numpy(), covering=rmdist._covering_view([a, b]).numel(),
                             separate=[t.numpy() for t in separate])
    finally:
        dist.destroy_process_group()


def test_two_rank_view_parallel_and_band_split(oracle):
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    pts, tets, cell = _scene()
    # serial reference: sum of the four views' gradients
    vg_ref = cg_ref = None
    for v in range(4):
        _, vg, cg, _, _ = _oracle_render_backward(oracle, pts, tets, cell, _view(v))
        vg_ref = vg if vg_ref is None else vg_ref + vg
        cg_ref = cg if cg_ref is None else cg_ref + cg
    for r in range(world):
        assert results[r]["n_images"] == 2
        np.testing.assert_allclose(results[r]["vg"], vg_ref, rtol=1e-5, atol=1e-5 * np.abs(vg_ref).max())
        np.testing.assert_allclose(results[r]["cg"], cg_ref, rtol=1e-5, atol=1e-5 * np.abs(cg_ref).max())
    # one view on two ranks: both ranks end with that view's gradients
    _, vg2, cg2, _, _ = _oracle_render_backward(oracle, pts, tets, cell, _view(2))
    for r in range(world):
        assert results[r]["n_images1"] == (1 if r == 0 else 0) and results[r]["raised"]
        np.testing.assert_allclose(results[r]["vg1"], vg2, rtol=1e-5, atol=1e-5 * np.abs(vg2).max())
        np.testing.assert_allclose(results[r]["cg1"], cg2, rtol=1e-5, atol=1e-5 * np.abs(cg2).max())
    for r in range(world):
        assert results[r]["mm_ok"] is False and results[r]["mm_reason"] and results[r]["mm_alloc_none"]
    # band split: the combined image equals the single-rank image bit for bit
    full_ref, _, _, idx_full, ranges_full = _oracle_render_backward(oracle, pts, tets, cell, _view(0))
    np.testing.assert_array_equal(results[0]["full"], full_ref)
    np.testing.assert_array_equal(results[1]["full"], full_ref)
    b0, b1 = results[0]["band"], results[1]["band"]
    assert b0[0] == 0 and b0[1] == b1[0] and b1[1] == _view(0)["grid_height"]
    # weights are the per-row key counts
    lens = (ranges_full[:, 1] - ranges_full[:, 0]).reshape(_view(0)["grid_height"], -1).sum(1)
    np.testing.assert_array_equal(results[0]["weights"], lens)
    # shared-allocation gradients: one collective over the covering view (ranks hold 1x and 2x the ramp)
    for r in range(2):
        assert results[r]["covering"] == 15
        np.testing.assert_array_equal(results[r]["flat"][:15], 3.0 * np.arange(15, dtype=np.float32))
        np.testing.assert_array_equal(results[r]["flat"][15:], (r + 1.0) * np.arange(15, 20, dtype=np.float32))
        np.testing.assert_array_equal(results[r]["separate"][0], np.full((3,), 3.0, np.float32))
        np.testing.assert_array_equal(results[r]["separate"][1], np.full((2, 2), 30.0, np.float32))


def test_band_lists_are_subsets_of_full_lists(oracle):
    pts, tets, cell = _scene()
    tcam = _view(1)
    pr = oracle.project(tets, pts, tcam)
    idx, ranges = oracle.build_lists(pr["tiles_touched"], pr["rect"], pr["vs_tetra"], tcam["grid_height"],
                                     tcam["grid_width"])
    gw = tcam["grid_width"]
    for band in rmdist.tile_row_bands(tcam["grid_height"], 3):
        tt, rect = oracle.restrict_to_tile_rows(pr["tiles_touched"], pr["rect"], *band)
        bidx, branges = oracle.build_lists(tt, rect, pr["vs_tetra"], tcam["grid_height"], gw)
        for t in range(band[0] * gw, band[1] * gw):
            np.testing.assert_array_equal(bidx[branges[t, 0]:branges[t, 1]], idx[ranges[t, 0]:ranges[t, 1]])
        outside = np.ones(len(branges), bool)
        outside[band[0] * gw:band[1] * gw] = False
        assert not branges[outside].any()


def test_tile_row_bands_partition():
    for gh, world in [(270, 8), (7, 3), (2, 4), (540, 8)]:
        bands = rmdist.tile_row_bands(gh, world)
        assert bands[0][0] == 0 and bands[-1][1] == gh
        assert all(bands[k][1] == bands[k + 1][0] for k in range(world - 1))
    w = np.zeros(100)
    w[40:60] = 1.0
    bands = rmdist.tile_row_bands(100, 4, w)
    sums = [w[a:b].sum() for a, b in bands]
    assert max(sums) - min(sums) <= 1.0 and sum(sums) == 20


def test_row_weights_from_walk_balance_bands():
    """Band weights from the previous frame: walk lengths blended with pair counts, normalised."""
    H, W, th, gh = 22, 8, 4, 6                      # a ragged last tile row (22 = 5*4 + 2)
    nc = torch.zeros((H, W, 1), dtype=torch.int32)
    nc[4:8] = 10                                    # tile row 1 walks a lot
    nc[20:22] = 5                                   # the ragged row a little
    rect = torch.tensor([[0, 0, 2, 1], [0, 1, 2, 3], [0, 5, 1, 6], [0, 0, 0, 0]], dtype=torch.int32)
    tt = torch.tensor([2, 4, 1, 0], dtype=torch.int32)
    w = rmdist.row_weights_from_walk(nc, rect, tt, gh, th, walk_share=0.75).numpy()
    assert w.shape == (gh,) and abs(w.sum() - 1.0) < 1e-12
    walk = np.array([0, 10 * 4 * W, 0, 0, 0, 5 * 2 * W], float)
    pairs = np.array([2, 2, 2, 0, 0, 1], float)
    np.testing.assert_allclose(w, 0.75 * walk / walk.sum() + 0.25 * pairs / pairs.sum(), rtol=1e-12)
    bands = rmdist.tile_row_bands(gh, 2, w)
    assert bands[0][1] <= 2                         # the heavy row ends the first band early
    # with the previous frame's hit counts: 4 * entries examined + 90 * entries evaluated per tile
    counts = torch.zeros((gh, 2), dtype=torch.int32)  # two tiles per row (W = 8, tile 4), one unit per tile
    counts[1] = torch.tensor([3, 1])
    counts[5] = torch.tensor([0, 2])
    w2 = rmdist.row_weights_from_walk(nc, rect, tt, gh, th, walk_share=0.75, hit_counts=counts.reshape(-1),
                                      tile_width=4).numpy()
    walk2 = np.array([0, 4 * 20 + 90 * 4, 0, 0, 0, 4 * 10 + 90 * 2], float)
    np.testing.assert_allclose(w2, 0.75 * walk2 / walk2.sum() + 0.25 * pairs / pairs.sum(), rtol=1e-12)


def test_overlapped_gradient_sum_is_inert_without_a_process_group():
    s = rmdist.OverlappedGradientSum(chunks=3)
    t = torch.ones(4)
    s(t)                                            # no process group: nothing happens, no CUDA needed
    s.done()
    assert torch.equal(t, torch.ones(4)) and s.comm is None


def test_multimem_gradient_sum_is_inert_without_a_process_group():
    """Without a process group (or before prepare()) it owns no buffer: the backward pass allocates as
    usual, ranges pass through untouched and export() hands the same tensor back."""
    s = rmdist.MultimemGradientSum(chunks=2)
    assert s.allocate(16, torch.device("cpu")) is None
    t = torch.ones(8)
    s(t)
    s.done()
    assert s.export(t) is t and torch.equal(t, torch.ones(8)) and s.comm is None


def test_pixel_hits_per_unit_reads_the_hit_list_layout():
    """Mask slots of unit q start at start(tile)*S + s*len(tile) + 16*q, 16 per batch of 16 recorded entries."""
    ranges = torch.tensor([[0, 5], [5, 45], [0, 0]], dtype=torch.int32)      # three tiles, one unit each
    counts = torch.tensor([3, 20, 0], dtype=torch.int32)                    # 1 batch, 2 batches, none
    masks = torch.full((45 + 16 * 3,), 0x7FFF, dtype=torch.int16)           # unwritten slots hold anything
    masks[0 + 0:0 + 16] = 0
    masks[0] = 0b0101                                                        # tile 0: two hits of pixel 0
    masks[3] = 0b0001
    b1 = 5 + 16 * 1
    masks[b1:b1 + 32] = 0
    masks[b1 + 2] = -1                                                       # 0xFFFF: 16 hits
    masks[b1 + 16 + 15] = 0b0100_0000_0000_0001
    got = rmdist.pixel_hits_per_unit(counts, masks, ranges)
    assert got.tolist() == [3, 18, 0]


def test_rebalance_bands_moves_rows_from_the_slow_rank():
    w = np.ones(100)
    bands = rmdist.tile_row_bands(100, 4, w)
    assert bands == [(0, 25), (25, 50), (50, 75), (75, 100)]
    new = rmdist.rebalance_bands(bands, [1.0, 3.0, 1.0, 1.0], w)     # rank 1 took three times as long
    assert new[0][0] == 0 and new[-1][1] == 100 and all(new[k][1] == new[k + 1][0] for k in range(3))
    assert new[1][1] - new[1][0] < 25 and new[0][1] > 25               # its band shrinks, its neighbours grow
    # time per row: 0.04, 0.12, 0.04, 0.04 -> total 6; cuts at 1.5, 3.0, 4.5 -> rows 30, 42.5, 62.5
    for (a, b), (ea, eb) in zip(new, [(0, 30), (30, 42), (42, 63), (63, 100)]):
        assert abs(a - ea) <= 1 and abs(b - eb) <= 1
    same = rmdist.rebalance_bands(bands, [1.0, 1.0, 1.0, 1.0], w)
    assert all(abs(a - ea) <= 1 and abs(b - eb) <= 1 for (a, b), (ea, eb) in zip(same, bands))
