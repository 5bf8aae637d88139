"""Layout vocabulary of GemmKernels.jl (src/layout.jl) as tags the C-ABI descriptor is built from.

In the reference a Layout is device code (logical tile -> address).  Here a layout only *names*
how an operand sits in memory; the kernels turn it into TMA tensor maps (aligned layouts), into
predicated loads (ColMajor / RowMajor), into "do not read" (Zero) or into a plane pair (Split*).
`Layout.ColMajor[Float16]` and `Layout.ColMajor(Float16)` both build the parametrised tag, standing
for Julia's `Layout.ColMajor{Float16}`.
"""
from __future__ import annotations

from .eltypes import ElType


class LayoutTag:
    """A parametrised layout, e.g. UnsafeAlignedColMajor{Float16} or Padded{L, 8}."""
    kind = "LayoutBase"
    col_major = True      # is the first logical index the contiguous one?
    aligned = False       # UnsafeAligned*: 16-byte aligned columns, sizes are tile multiples
    zero = False
    diagonal = False
    split = False         # planar complex (plane is the last dimension)
    interleaved = False   # Complex{T} pairs

    def __init__(self, eltype: ElType):
        self.eltype = eltype

    def __class_getitem__(cls, eltype):
        return cls(eltype)

    def __eq__(self, other):
        return type(self) is type(other) and self.__dict__ == other.__dict__

    def __hash__(self):
        return hash((type(self).__name__, tuple(sorted((k, repr(v)) for k, v in self.__dict__.items()))))

    def __repr__(self):
        return f"Layout.{self.kind}{{{self.eltype}}}"

    # src/layout.jl:76 — physical_size defaults to the logical size
    def physical_size(self, logical_size):
        return tuple(logical_size)

    @property
    def base(self) -> "LayoutTag":
        return self


class Zero(LayoutTag):            # src/layout.jl:82-89
    kind = "Zero"; zero = True


class ColMajor(LayoutTag):        # src/layout.jl:111-144 (bounds-checked)
    kind = "ColMajor"


class RowMajor(LayoutTag):        # src/layout.jl:150-184 (bounds-checked)
    kind = "RowMajor"; col_major = False


class UnsafeAlignedColMajor(LayoutTag):   # src/layout.jl:192-219
    kind = "UnsafeAlignedColMajor"; aligned = True


class UnsafeAlignedRowMajor(LayoutTag):   # src/layout.jl:244-270
    kind = "UnsafeAlignedRowMajor"; aligned = True; col_major = False


class Diagonal(LayoutTag):        # src/layout.jl:225-236
    kind = "Diagonal"; diagonal = True; aligned = True


class InterleavedColMajor(LayoutTag):     # src/layout.jl:276-303
    kind = "InterleavedColMajor"; interleaved = True


class InterleavedRowMajor(LayoutTag):     # src/layout.jl:305-334
    kind = "InterleavedRowMajor"; interleaved = True; col_major = False


class SplitColMajor(LayoutTag):   # src/layout.jl:340-373
    kind = "SplitColMajor"; split = True

    def physical_size(self, logical_size):
        return (*tuple(logical_size), 2)


class SplitRowMajor(LayoutTag):   # src/layout.jl:379-411
    kind = "SplitRowMajor"; split = True; col_major = False

    def physical_size(self, logical_size):
        return (*tuple(logical_size), 2)


class Padded(LayoutTag):
    """Padded{L, P} (src/layout.jl:95-105).  Padding only existed to dodge shared-memory bank
    conflicts; the 128-byte swizzle does that here, so the tag is kept for API and heuristics."""
    kind = "Padded"

    def __init__(self, inner: LayoutTag, pad: int):
        self.inner = inner
        self.pad = int(pad)
        self.eltype = inner.eltype

    def __class_getitem__(cls, args):
        inner, pad = args
        return cls(inner, pad)

    def __repr__(self):
        return f"Layout.Padded{{{self.inner!r}, {self.pad}}}"

    # col_major / aligned / ... are those of the wrapped layout
    col_major = property(lambda self: self.inner.col_major)
    aligned = property(lambda self: self.inner.aligned)
    zero = property(lambda self: self.inner.zero)
    diagonal = property(lambda self: self.inner.diagonal)
    split = property(lambda self: self.inner.split)
    interleaved = property(lambda self: self.inner.interleaved)

    @property
    def base(self):
        return self.inner.base

    def physical_size(self, logical_size):
        s = tuple(logical_size)
        # src/layout.jl:196 / 246: the pad goes on the contiguous dimension
        if not self.inner.col_major:
            return (s[1] + self.pad, s[0])
        return (s[0] + self.pad, *s[1:])


