"""Transform vocabulary (src/transform.jl:19-30).

The reference lets any Julia functor run at eight hook points.  A functor cannot cross a C ABI, so
this engine takes a closed set of named functors and folds each hook into the fused epilogue
(alpha, beta, activation).  Anything else raises UnsupportedFunctor — there is no CPU fallback.
"""
from __future__ import annotations


class Functor:
    def __eq__(self, other):
        return type(self) is type(other) and self.__dict__ == other.__dict__

    def __hash__(self):
        return hash((type(self).__name__, tuple(self.__dict__.items())))


class Identity(Functor):
    def __repr__(self):
        return "identity"


class Scale(Functor):
    """x -> x * factor (what `matmatmul!` builds for alpha and beta, src/matmul.jl:199-200)."""

    def __init__(self, factor):
        self.factor = factor

    def __repr__(self):
        return f"Scale({self.factor})"


class ReLU(Functor):
    def __repr__(self):
        return "ReLU()"


class GELU(Functor):
    def __repr__(self):
        return "GELU()"


class Cast(Functor):
    """Convert to the element type of D; the store already does this, so it folds to nothing."""

    def __init__(self, eltype):
        self.eltype = eltype

    def __repr__(self):
        return f"Cast({self.eltype})"


class UnsupportedFunctor(Exception):
    pass


class Elementwise:
    """Transform.Elementwise(f): f must be one of the functors above (or None / `identity`)."""

    def __init__(self, f=None):
        if f is None:
            f = Identity()
        if callable(f) and not isinstance(f, Functor):
            raise UnsupportedFunctor(
                f"Transform.Elementwise got {f!r}: only identity, Scale, ReLU, GELU and Cast are "
                "compiled into the kernels; arbitrary functions are rejected (no CPU fallback)")
        if not isinstance(f, Functor):
            raise UnsupportedFunctor(f"Transform.Elementwise got {f!r}, not a functor")
        self.f = f

    def __repr__(self):
        return f"Transform.Elementwise({self.f!r})"
