"""Tile-grid geometry (mirrors delaunay_rasterization/internal/render_grid.py:17-27)."""


def ceil_div(x, y):
    return -(-x // y)


class RenderGrid:
    """Image size, tile size and the resulting number of tiles per axis.

    Argument order is (image_height, image_width, tile_width, tile_height), as in
    the reference; callers there pass the tile sizes by keyword.
    """

    def __init__(self, image_height, image_width, tile_width, tile_height):
        self.image_height = image_height
        self.image_width = image_width
        self.tile_height = tile_height
        self.tile_width = tile_width
        self.grid_height = ceil_div(image_height, tile_height)
        self.grid_width = ceil_div(image_width, tile_width)
