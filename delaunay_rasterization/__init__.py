"""Drop-in replacement for the reference's `delaunay_rasterization` package.

Same module paths and call signatures as the reference
(delaunay_rasterization/internal/*.py), backed by the sm_100a CUDA library of
`radiance_meshes_b200` instead of Slang-generated kernels.
"""
__version__ = "0.1.0"
