"""Epilogue vocabulary (src/epilogue.jl)."""
from __future__ import annotations


class Default:                    # src/epilogue.jl:14-34
    def __repr__(self):
        return "Epilogue.Default()"


class Bias:
    """Epilogue.Bias(pointer(bias)) (src/epilogue.jl:40-73): Float32 bias added after the
    regs_to_shared_d transform and before shared_to_global_d.  The reference indexes it by column
    (length N); `axis="row"` selects one value per row (length M) instead."""

    def __init__(self, bias, axis: str = "col"):
        if axis not in ("col", "row"):
            raise ValueError("axis must be 'col' or 'row'")
        self.bias = bias
        self.axis = axis

    def __repr__(self):
        return f"Epilogue.Bias(<{self.axis}>)"
