"""Element types of the GemmKernels.jl vocabulary and their C-ABI / torch / numpy counterparts."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _lib as L


@dataclass(frozen=True)
class ElType:
    """A Julia element type name with its size and the ids the other layers use for it."""
    name: str
    size: int            # bytes per (real) element
    gk: int              # gk_dtype of the real component
    np_dtype: object     # numpy dtype of the real component (None when numpy has none)
    torch_name: str      # attribute name in torch
    is_complex: bool = False
    is_integer: bool = False

    def __repr__(self) -> str:
        return self.name

    @property
    def real(self) -> "ElType":
        return _REAL_OF.get(self.name, self)

    def torch_dtype(self):
        import torch
        return getattr(torch, self.torch_name)


Float16 = ElType("Float16", 2, L.GK_F16, np.float16, "float16")
BFloat16 = ElType("BFloat16", 2, L.GK_BF16, None, "bfloat16")
Float32 = ElType("Float32", 4, L.GK_F32, np.float32, "float32")
Float64 = ElType("Float64", 8, L.GK_F64, np.float64, "float64")
Int16 = ElType("Int16", 2, L.GK_I16, np.int16, "int16", is_integer=True)
Int32 = ElType("Int32", 4, L.GK_I32, np.int32, "int32", is_integer=True)
Int64 = ElType("Int64", 8, L.GK_I64, np.int64, "int64", is_integer=True)
# Complex{T}: stored as (re, im) pairs of T.  Dual numbers reuse the same storage
# (configs/configs.jl:136-140 reinterprets Complex as ForwardDiff.Dual for verification only).
ComplexF16 = ElType("Complex{Float16}", 2, L.GK_F16, np.float16, "float16", is_complex=True)
ComplexF32 = ElType("Complex{Float32}", 4, L.GK_F32, np.float32, "float32", is_complex=True)

_REAL_OF = {"Complex{Float16}": Float16, "Complex{Float32}": Float32}
_BY_TORCH = {t.torch_name: t for t in (Float16, BFloat16, Float32, Float64, Int16, Int32, Int64)}

_PROMOTE_ORDER = [Int16, Int32, Int64, Float16, BFloat16, Float32, Float64]


def from_torch(dtype) -> ElType:
    name = str(dtype).replace("torch.", "")
    if name not in _BY_TORCH:
        raise TypeError(f"no GemmKernels element type for torch dtype {dtype}")
    return _BY_TORCH[name]


def promote_type(a: ElType, b: ElType) -> ElType:
    """Julia's promote_type restricted to the types above (same type -> itself)."""
    if a == b:
        return a
    ia, ib = _PROMOTE_ORDER.index(a.real), _PROMOTE_ORDER.index(b.real)
    return _PROMOTE_ORDER[max(ia, ib)]
