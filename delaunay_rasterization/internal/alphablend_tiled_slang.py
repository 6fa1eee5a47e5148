"""Constant-colour debug renderer, drop-in for the reference module of the same name
(delaunay_rasterization/internal/alphablend_tiled_slang.py:16-192).

`render_constant_color` is what utils/train_util.py:164-186 (`render_debug`) calls to turn
a per-tet scalar or colour into an image.  `AlphaBlendTiledRender` is differentiable in the
vertices and in rgbs, with the reference's formulation of the backward pass
(slang/alphablend_shader.slang:186-277).
"""
import torch

from delaunay_rasterization.internal.render_grid import RenderGrid
from delaunay_rasterization.internal.tile_shader_slang import lookup_tiles_touched, vertex_and_tile_shader
from radiance_meshes_b200 import _lib, raster


class AlphaBlendTiledRender(torch.autograd.Function):
    """apply(sorted_tetra_idx, tile_ranges, indices, vertices, rgbs[T,4] = (r,g,b,density), render_grid, tcam,
    pre_multi, ladder_p) -> (output_img[H,W,4] = (r,g,b,transmittance), distortion_img[H,W,4])."""

    @staticmethod
    def forward(ctx, sorted_tetra_idx, tile_ranges, indices, vertices, rgbs, render_grid, tcam, pre_multi, ladder_p,
                device="cuda"):
        dev = vertices.device
        raster._require_cuda(vertices, "vertices")
        cam = raster.CameraArgs(tcam, dev)
        assert cam.c.grid_height == render_grid.grid_height and cam.c.grid_width == render_grid.grid_width
        rgbs = rgbs.detach().float()
        assert rgbs.shape[1] == 4, "rgbs are (r, g, b, density) per tet"
        T = indices.shape[0]
        # records of the interpolating renderer with a zero colour gradient: (density, r, g, b, 0, 0, 0)
        cell = torch.cat([rgbs[:, 3:4], rgbs[:, :3], torch.zeros((T, 3), device=dev)], dim=1).contiguous()
        records = raster.pack_records(indices, vertices.detach().contiguous().float(), cell, cam,
                                      lookup_tiles_touched(sorted_tetra_idx))
        H, W = render_grid.image_height, render_grid.image_width
        lib = _lib.load()
        with torch.cuda.device(dev):
            output_img = torch.empty((H, W, 4), dtype=torch.float32, device=dev)
            distortion_img = torch.empty((H, W, 4), dtype=torch.float32, device=dev)
            n_contributors = torch.empty((H, W, 1), dtype=torch.int32, device=dev)
            _lib.check(lib.rm_forward_constant_color(
                raster._ptr(sorted_tetra_idx), raster._ptr(tile_ranges), raster._ptr(records), cam.ref,
                float(pre_multi), float(ladder_p), raster._ptr(output_img), raster._ptr(distortion_img),
                raster._ptr(n_contributors), raster._stream(dev)))
        ctx.save_for_backward(sorted_tetra_idx, tile_ranges, indices, vertices.detach().contiguous().float(), cell,
                              records, output_img, distortion_img, n_contributors)
        ctx.cam = cam
        ctx.scalars = (float(pre_multi), float(ladder_p))
        return output_img, distortion_img

    @staticmethod
    def backward(ctx, grad_output_img, grad_distortion_img):
        (sorted_tetra_idx, tile_ranges, indices, verts, cell, records, output_img, distortion_img,
         n_contributors) = ctx.saved_tensors
        dev = verts.device
        T, V = indices.shape[0], verts.shape[0]
        pre_multi, ladder_p = ctx.scalars
        lib = _lib.load()
        idx32 = indices.contiguous().to(torch.int32)
        g_img = grad_output_img.contiguous().float()
        g_dist = grad_distortion_img.contiguous().float()
        with torch.cuda.device(dev):
            grad_records = torch.empty((T, _lib.RM_GRAD_RECORD_FLOATS), dtype=torch.float32, device=dev)
            flags = torch.empty((max(T, 1),), dtype=torch.uint8, device=dev)
            vertices_grad = torch.empty((V, 3), dtype=torch.float32, device=dev)
            cell_grad = torch.empty((T, 7), dtype=torch.float32, device=dev)
            if _lib.bounds_checked():
                _lib.set_extents(list=sorted_tetra_idx.shape[0], tets=T, verts=V)
            _lib.check(lib.rm_backward_constant_color(
                raster._ptr(sorted_tetra_idx), raster._ptr(tile_ranges), raster._ptr(records), ctx.cam.ref, pre_multi,
                ladder_p, raster._ptr(output_img), raster._ptr(distortion_img), raster._ptr(n_contributors),
                raster._ptr(g_img), raster._ptr(g_dist), raster._ptr(idx32), raster._ptr(verts), raster._ptr(cell), T, V,
                raster._ptr(grad_records), raster._ptr(flags), raster._ptr(vertices_grad), raster._ptr(cell_grad),
                raster._stream(dev)))
        rgbs_grad = torch.cat([cell_grad[:, 1:4], cell_grad[:, 0:1]], dim=1)
        return None, None, None, vertices_grad, rgbs_grad, None, None, None, None


def render_constant_color(indices, vertices, rgbs_fn, camera, cell_values=None, tile_size=16, min_t=0.1):
    """Same arguments and result dictionary as the reference's function
    (alphablend_tiled_slang.py:16-80).  As there, `cell_values` ([T,4]: r, g, b, density) is what is
    rendered; `rgbs_fn` is accepted and, as in the reference (its result is overwritten at :53),
    not used."""
    device = indices.device
    if cell_values is None:
        raise ValueError("render_constant_color needs cell_values [T,4] = (r, g, b, density)")
    render_grid = RenderGrid(camera.image_height, camera.image_width, tile_height=tile_size, tile_width=tile_size)
    tcam = dict(tile_height=tile_size, tile_width=tile_size, grid_height=render_grid.grid_height,
                grid_width=render_grid.grid_width, min_t=min_t, **camera.to_dict(device))
    sorted_tetra_idx, tile_ranges, vs_tetra, circumcenter, mask, _ = vertex_and_tile_shader(
        indices, vertices, tcam, render_grid)
    rgbs = cell_values
    image_rgb, distortion_img = AlphaBlendTiledRender.apply(
        sorted_tetra_idx, tile_ranges, indices, vertices, rgbs, render_grid, tcam, 100, -0.1)
    return {
        "render": image_rgb.permute(2, 0, 1)[:3, ...],
        "viewspace_points": vs_tetra,
        "visibility_filter": mask,
        "circumcenters": circumcenter,
        "rgbs": rgbs,
        "mask": mask,
    }
