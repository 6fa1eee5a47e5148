"""Stages 5-6 behind the reference's entry point
(delaunay_rasterization/internal/alphablend_tiled_slang_interp.py:10-112).

AlphaBlendTiledRender.apply(sorted_tetra_idx, tile_ranges, indices, vertices,
tet_density, render_grid, tcam, ray_jitter) -> (output_img[H,W,4],
distortion_img[H,W,5], tet_alive[T] bool); backward returns gradients for
`vertices` and `tet_density` only.  Any tile size is accepted (the reference
compiles 4x4 only).
"""
import torch

from delaunay_rasterization.internal.render_grid import RenderGrid  # noqa: F401  (re-exported by the reference)
from delaunay_rasterization.internal.tile_shader_slang import lookup_tiles_touched, vertex_and_tile_shader  # noqa: F401
from radiance_meshes_b200 import raster


class AlphaBlendTiledRender(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sorted_tetra_idx, tile_ranges, indices, vertices, tet_density, render_grid, tcam, ray_jitter,
                device="cuda"):
        dev = vertices.device
        indices = indices.contiguous()
        if indices.dtype != torch.int32:
            indices = indices.to(torch.int32)
        verts = vertices.detach().contiguous().float()
        cell = tet_density.detach().contiguous().float()
        jitter = ray_jitter.detach().contiguous().float()
        assert cell.shape[1] == 7, "cell values are (density, r, g, b, gx, gy, gz) per tet"
        assert jitter.shape == (render_grid.image_height, render_grid.image_width, 2)
        cam = raster.CameraArgs(tcam, dev)
        assert cam.c.grid_height == render_grid.grid_height and cam.c.grid_width == render_grid.grid_width
        records = raster.pack_records(indices, verts, cell, cam, lookup_tiles_touched(sorted_tetra_idx))
        need_grad = vertices.requires_grad or tet_density.requires_grad
        output_img, distortion_img, n_contributors, hits = raster.forward(
            sorted_tetra_idx, tile_ranges, records, cam, jitter, want_hit_masks=need_grad)
        if hits is None:  # nothing to differentiate: backward is never called
            hits = tuple(torch.empty((0,), dtype=dt, device=dev)
                         for dt in (torch.int32, torch.int32, torch.int16, torch.uint8))
        # never written by the reference kernel either: always False
        tet_alive = torch.zeros((indices.shape[0],), dtype=torch.bool, device=dev)
        ctx.save_for_backward(sorted_tetra_idx, tile_ranges, indices, verts, cell, output_img, distortion_img,
                              n_contributors, jitter, records, *hits)
        ctx.cam = cam
        ctx.mark_non_differentiable(tet_alive)
        return output_img, distortion_img, tet_alive

    @staticmethod
    def backward(ctx, grad_output_img, grad_distortion_img, grad_vert_alive):
        (sorted_tetra_idx, tile_ranges, indices, verts, cell, output_img, distortion_img, n_contributors, jitter,
         records, hit_counts, hit_ids, hit_masks, tet_flags) = ctx.saved_tensors
        vertices_grad, cell_grad = raster.backward(
            sorted_tetra_idx, tile_ranges, records, ctx.cam, jitter, output_img, distortion_img, n_contributors,
            (hit_counts, hit_ids, hit_masks, tet_flags), grad_output_img.contiguous().float(),
            grad_distortion_img.contiguous().float(), indices, verts, cell)
        return None, None, None, vertices_grad, cell_grad, None, None, None
