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


def _even_bits(x: int) -> int:
    out, bit = 0, 0
    while x:
        out |= (x & 1) << bit
        x >>= 2
        bit += 1
    return out


def tile_of(swizzle, t: int, tiles_m: int, tiles_n: int, group: int = 0):
    """(tile_m, tile_n) the persistent scheduler visits at step t: the host mirror of the kernel's
    tile walk.  Tiled swizzles walk bands of T tiles (down M for VerticallyTiled and by default, along
    N for HorizontallyTiled); LebesgueCurve follows the Z-order curve (M takes the even bits,
    src/cta-swizzle.jl:155-158) on power-of-two grids and the default bands elsewhere."""
    pow2 = lambda x: x > 0 and x & (x - 1) == 0
    if isinstance(swizzle, LebesgueCurve) and pow2(tiles_m) and pow2(tiles_n):
        zb = min(tiles_m.bit_length(), tiles_n.bit_length()) - 1
        low, rest = t & ((1 << (2 * zb)) - 1), t >> (2 * zb)
        tm, tn = _even_bits(low), _even_bits(low >> 1)
        return (tm + (rest << zb), tn) if tiles_m >= tiles_n else (tm, tn + (rest << zb))
    along_n = isinstance(swizzle, HorizontallyTiled)
    major, minor = (tiles_n, tiles_m) if along_n else (tiles_m, tiles_n)
    g = major if isinstance(swizzle, Identity) else (getattr(swizzle, "tile", 0) or group or 8)
    g = max(1, min(g, major))
    band = g * minor
    band_id = t // band
    first = band_id * g
    rows = min(g, major - first)
    r = t - band_id * band
    a, b = first + r % rows, r // rows
    return (b, a) if along_n else (a, b)


def visualise_cta_swizzle(swizzle, tiles_m: int, tiles_n: int):
    """tiles_m x tiles_n table of the order in which the persistent scheduler visits tiles."""
    order = [[-1] * tiles_n for _ in range(tiles_m)]
    for t in range(tiles_m * tiles_n):
        tm, tn = tile_of(swizzle, t, tiles_m, tiles_n)
        order[tm][tn] = t
    return order
