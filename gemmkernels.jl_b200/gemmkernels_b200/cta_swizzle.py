"""CTASwizzle vocabulary (src/cta-swizzle.jl:26-160) as raster orders of the persistent scheduler."""
from __future__ import annotations

from . import _lib as L


class _Swizzle:
    raster = L.GK_RASTER_AUTO
    tile = 0

    def __eq__(self, other):
        return type(self) is type(other) and self.tile == other.tile

    def __hash__(self):
        return hash((type(self).__name__, self.tile))

    def __repr__(self):
        return f"CTASwizzle.{type(self).__name__}" + (f"{{{self.tile}}}" if self.tile else "")


class Identity(_Swizzle):                 # src/cta-swizzle.jl:26-41
    raster = L.GK_RASTER_IDENTITY


class _Tiled(_Swizzle):
    def __init__(self, tile: int = 8):
        self.tile = int(tile)

    def __class_getitem__(cls, tile):
        return cls(tile)


class HorizontallyTiled(_Tiled):          # src/cta-swizzle.jl:47-90
    raster = L.GK_RASTER_HORIZONTAL


class VerticallyTiled(_Tiled):            # src/cta-swizzle.jl:92-130
    raster = L.GK_RASTER_VERTICAL


class LebesgueCurve(_Swizzle):            # src/cta-swizzle.jl:132-160
    raster = L.GK_RASTER_LEBESGUE


def _cld(a, b):
    return -(-a // b)


def number_of_blocks(swizzle, block_shape, matmul_shape):
    """Grid the reference would launch (src/cta-swizzle.jl:28-31 and the tiled variants)."""
    return (_cld(matmul_shape["M"], block_shape["M"]), _cld(matmul_shape["N"], block_shape["N"]))


def visualise_cta_swizzle(swizzle, tiles_m: int, tiles_n: int):
    """tiles_m x tiles_n table of the order in which the persistent scheduler visits tiles."""
    group = tiles_m if isinstance(swizzle, Identity) else (getattr(swizzle, "tile", 0) or 8)
    group = max(1, min(group, tiles_m))
    order = [[0] * tiles_n for _ in range(tiles_m)]
    for t in range(tiles_m * tiles_n):
        band = group * tiles_n
        band_id = t // band
        first_m = band_id * group
        rows = min(group, tiles_m - first_m)
        r = t - band_id * band
        order[first_m + r % rows][r // rows] = t
    return order
