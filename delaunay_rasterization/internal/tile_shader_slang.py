"""Stages 1-4 behind the reference's entry points
(delaunay_rasterization/internal/tile_shader_slang.py:24-150).

`vertex_and_tile_shader` returns exactly what the reference returns:
(sorted_tetra_idx[N] i32, tile_ranges[G,2] i32, vs_tetra[T,3], circumcenter[T,3],
mask[T] bool, rect_tile_space[T,4] i32), with autograd from vs_tetra and
circumcenter to the vertices.  One host synchronisation (to learn N) instead of
the reference's four.
"""
import torch

from radiance_meshes_b200 import raster


def ceil_div(x, y):
    return -(-x // y)


def lookup_tiles_touched(sorted_tetra_idx):
    """tiles_touched of the call that produced this list tensor (None for any other tensor): the
    integration stage skips the records of culled tets with it."""
    return getattr(sorted_tetra_idx, "_rm_tiles_touched", None)


class VertexShader(torch.autograd.Function):
    """Per-tet projection, culling, sort depth, circumcentre and tile count.

    `holder`, if given, receives the binning context (workspace, tile ranges, counters) that
    `vertex_and_tile_shader` needs to finish the tile lists; a bare `VertexShader.apply(indices,
    vertices, tcam, render_grid)` keeps nothing beyond its four outputs."""

    @staticmethod
    def forward(ctx, indices, vertices, tcam, render_grid, *extra):
        # extra: the reference's optional `device` argument, then the optional holder
        holder = extra[1] if len(extra) > 1 else None
        ctx.n_extra = len(extra)
        bctx = raster.project_and_bin(indices, vertices, tcam)
        ctx.bctx_small = (bctx["indices"], bctx["vertices"], bctx["cam"], bctx["tiles_touched"])
        ctx.mark_non_differentiable(bctx["tiles_touched"], bctx["rect"])
        if holder is not None:
            holder["bctx"] = bctx
        return bctx["tiles_touched"], bctx["rect"], bctx["vs_tetra"], bctx["circumcenter"]

    @staticmethod
    def backward(ctx, grad_tiles_touched, grad_rect_tile_space, grad_vs_tetra, grad_circumcenter):
        indices, vertices, cam, tiles_touched = ctx.bctx_small
        grad_vertices = raster.vertex_backward(indices, vertices, cam, tiles_touched,
                                               grad_vs_tetra.contiguous().float(),
                                               grad_circumcenter.contiguous().float())
        return (None, grad_vertices, None, None) + (None,) * ctx.n_extra


def vertex_and_tile_shader(indices, vertices, cam, render_grid):
    holder = {}
    tiles_touched, rect_tile_space, vs_tetra, circumcenter = VertexShader.apply(indices, vertices, cam, render_grid,
                                                                                "cuda", holder)
    bctx = holder.pop("bctx")
    with torch.no_grad():
        n_keys, _ = raster.read_info(bctx)
        sorted_tetra_idx = raster.build_tile_lists(bctx, n_keys)
        tile_ranges = bctx["tile_ranges"]
        mask = tiles_touched > 0
    sorted_tetra_idx._rm_tiles_touched = tiles_touched
    return sorted_tetra_idx, tile_ranges, vs_tetra, circumcenter, mask, rect_tile_space
