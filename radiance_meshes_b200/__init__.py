"""B200-native differentiable tetrahedral tile rasterizer (hot path of radiance_meshes)."""
__version__ = "0.1.0"
