"""Densification statistics behind the reference's entry point
(delaunay_rasterization/internal/render_err.py:33-159).

render_err(gt_image, camera, model, tile_size, min_t) renders the view, forms the
per-pixel L1 and SSIM errors exactly as the reference does (in torch, with the
reference's own `utils.ssim.ssim`, which must be importable — it is when this
package is used inside the reference tree) and scatters the per-tet error moments
with the CUDA library instead of the Slang `calc_tet_err` kernel.
"""
import torch

from delaunay_rasterization.internal.render_grid import RenderGrid
from delaunay_rasterization.internal.tile_shader_slang import vertex_and_tile_shader
from radiance_meshes_b200 import raster


def tet_error_stats(sorted_tetra_idx, tile_ranges, indices, vertices, cell_values, tcam, pixel_err, ssim_err,
                    tiles_touched=None):
    """The kernel-level part: (tet_err[T,16] f32, tet_count[T,2] i32) for given per-pixel errors."""
    dev = vertices.device
    indices = indices.contiguous().to(torch.int32)
    verts = vertices.detach().contiguous().float()
    cell = cell_values.detach().contiguous().float()
    cam = raster.CameraArgs(tcam, dev)
    records = raster.pack_records(indices, verts, cell, cam, tiles_touched)
    return raster.tet_err(sorted_tetra_idx, tile_ranges, records, cam, pixel_err.detach().contiguous().float(),
                          ssim_err.detach().contiguous().float(), indices.shape[0])


def render_err(gt_image, camera, model, tile_size=16, min_t=0.1, **kwargs):
    from utils.ssim import ssim  # the reference's SSIM (utils/ssim.py); not part of this package
    device = model.device
    indices = model.indices
    vertices = model.vertices
    render_grid = RenderGrid(camera.image_height, camera.image_width, tile_height=tile_size, tile_width=tile_size)
    tcam = dict(tile_height=tile_size, tile_width=tile_size, grid_height=render_grid.grid_height,
                grid_width=render_grid.grid_width, min_t=min_t, **camera.to_dict(device))
    with torch.no_grad():
        sorted_tetra_idx, tile_ranges, vs_tetra, circumcenter, mask, _ = vertex_and_tile_shader(
            indices, vertices, tcam, render_grid)
        cell_values = torch.zeros((mask.shape[0], model.feature_dim), device=circumcenter.device)
        _, cell_values[mask] = model.get_cell_values(camera, mask)
        dev = vertices.device
        idx32 = indices.contiguous().to(torch.int32)
        verts = vertices.detach().contiguous().float()
        cam = raster.CameraArgs(tcam, dev)
        records = raster.pack_records(idx32, verts, cell_values.contiguous().float(), cam, mask.to(torch.int32))
        ray_jitter = 0.5 * torch.ones((camera.image_height, camera.image_width, 2), device=device)
        output_img, _, _, _ = raster.forward(sorted_tetra_idx, tile_ranges, records, cam, ray_jitter,
                                             want_hit_masks=False)
        render_img = output_img.permute(2, 0, 1)[:3, ...].clip(min=0, max=1)
        l1_err = (render_img - gt_image).mean(dim=0)
        ssim_err = (1 - ssim(render_img, gt_image).mean(dim=0)).clip(min=0, max=1)
        pixel_err = l1_err.contiguous()
        alpha_mask = camera.gt_alpha_mask.to(device)
        pixel_err = pixel_err * alpha_mask[0]
        ssim_err = ssim_err * alpha_mask[0]
        render_img = render_img * alpha_mask
        assert pixel_err.shape == (render_grid.image_height, render_grid.image_width)
        assert ssim_err.shape == (render_grid.image_height, render_grid.image_width)
        tet_err, tet_count = raster.tet_err(sorted_tetra_idx, tile_ranges, records, cam, pixel_err.contiguous(),
                                            ssim_err.contiguous(), idx32.shape[0])
    return tet_err, dict(tet_count=tet_count, pixel_err=pixel_err, ssim_err=ssim_err, render_img=render_img,
                         cell_values=cell_values)
