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


def render(indices, vertices, cell_values, tcam, ray_jitter=None):
    """Returns dict(render[3,H,W], alpha[H,W] (log-transmittance), distortion_loss, mask, image, distortion_img)."""
    H, W = int(tcam["image_height"]), int(tcam["image_width"])
    device = vertices.device
    if ray_jitter is None:
        ray_jitter = 0.5 * torch.ones((H, W, 2), device=device)
    grid = RenderGrid(H, W, tile_height=int(tcam["tile_height"]), tile_width=int(tcam["tile_width"]))
    sorted_tetra_idx, tile_ranges, vs_tetra, circumcenter, mask, rect = vertex_and_tile_shader(
        indices, vertices, tcam, grid)
    image, distortion_img, tet_alive = AlphaBlendTiledRender.apply(
        sorted_tetra_idx, tile_ranges, indices, vertices, cell_values, grid, tcam, ray_jitter)
    total_density = (distortion_img[:, :, 2] ** 2).clip(min=1e-6)
    distortion_loss = (((distortion_img[:, :, 0] - distortion_img[:, :, 1]) + distortion_img[:, :, 4])
                       / total_density).clip(min=0)
    return dict(render=image.permute(2, 0, 1)[:3], alpha=image[..., 3], distortion_loss=distortion_loss.mean(),
                mask=mask, image=image, distortion_img=distortion_img, sorted_tetra_idx=sorted_tetra_idx,
                tile_ranges=tile_ranges, vs_tetra=vs_tetra, circumcenter=circumcenter, rect=rect)
