"""Operator vocabulary (src/operator.jl).  An operator tag names the arithmetic of the inner loop;
the kernels behind the C ABI implement it.

  TCGen05Operator{CT, AT}            new: tcgen05.mma with TMEM accumulators; CT in Float16,
                                     BFloat16, TF32 (FP32 storage), AT = Float32 accumulate
  WMMAOp{M,N,K,CT,AT}                accepted for source compatibility, runs as TCGen05Operator
  WMMAComplexOp / WMMADualOp         planar complex / dual products (4 / 3 MMAs per step)
  FPUOp{M,N,K,mb,nb,kb,CT,AT}        FP32/FP64/integer FMA on the CUDA cores
  TropicalFPUOp{...}                 max-plus
"""
from __future__ import annotations

from .eltypes import ElType, Float16, Float32


class TF32Type:
    """Compute-type marker: Float32 storage multiplied as TF32 on the tensor cores."""
    name = "TF32"
    size = 4

    def __repr__(self):
        return "TF32"


TF32 = TF32Type()


class OperatorTag:
    kind = "Operator"
    tensor = False
    number = "real"       # real | complex | dual
    tropical = False

    def __eq__(self, other):
        return type(self) is type(other) and self.__dict__ == other.__dict__

    def __hash__(self):
        return hash((type(self).__name__, repr(sorted(self.__dict__.items(), key=lambda kv: kv[0]))))


class _ShapeOp(OperatorTag):
    def shape(self):
        return {"M": self.M, "N": self.N, "K": self.K}


class TCGen05Operator(OperatorTag):
    """Operator.TCGen05Operator{CT, AT}: one instruction covers 128 (or 256) x tile_n x (32 bytes
    of K).  `shape()` reports the granularity used by get_config's block-shape rules, chosen equal
    to the 16 x 16 x 16 WMMA shape for 16-bit types so that defaults match the reference's."""
    kind = "TCGen05Operator"; tensor = True

    def __init__(self, CT=Float16, AT=Float32, number: str = "real"):
        self.CT, self.AT, self.number = CT, AT, number

    def __class_getitem__(cls, args):
        return cls(*args) if isinstance(args, tuple) else cls(args)

    def shape(self):
        return {"M": 16, "N": 16, "K": 32 // self.CT.size}

    def __repr__(self):
        return f"Operator.TCGen05Operator{{{self.CT}, {self.AT}}}"


class WMMAOp(_ShapeOp):           # src/operator.jl:163-245
    kind = "WMMAOp"; tensor = True

    def __init__(self, M, N, K, CT=Float16, AT=Float32):
        self.M, self.N, self.K, self.CT, self.AT = M, N, K, CT, AT

    def __class_getitem__(cls, args):
        return cls(*args)

    def __repr__(self):
        return f"Operator.{self.kind}{{{self.M}, {self.N}, {self.K}, {self.CT}, {self.AT}}}"


class WMMAComplexOp(WMMAOp):      # src/operator.jl:251-314
    kind = "WMMAComplexOp"; number = "complex"


class WMMADualOp(WMMAOp):         # src/operator.jl:320-372
    kind = "WMMADualOp"; number = "dual"


class FPUOp(_ShapeOp):            # src/operator.jl:35-132
    kind = "FPUOp"

    def __init__(self, M, N, K, mb, nb, kb, CT, AT):
        self.M, self.N, self.K, self.mb, self.nb, self.kb, self.CT, self.AT = M, N, K, mb, nb, kb, CT, AT

    def __class_getitem__(cls, args):
        return cls(*args)

    def base_shape(self):
        return {"M": self.M, "N": self.N, "K": self.K, "mb": self.mb, "nb": self.nb, "kb": self.kb}

    def __repr__(self):
        return (f"Operator.{self.kind}{{{self.M}, {self.N}, {self.K}, {self.mb}, {self.nb}, {self.kb}, "
                f"{self.CT}, {self.AT}}}")


class TropicalFPUOp(FPUOp):       # src/operator.jl:134-137
    kind = "TropicalFPUOp"; tropical = True
