"""Device arrays in Julia (column-major) order on top of torch tensors.

A Julia `CuArray{T,2}` of size (r, c) is a torch CUDA tensor of shape (r, c) with strides (1, ld),
ld >= r.  Planar complex / dual operands (Layout.Split*) are (r, c, 2) with strides (1, ld, plane).
Interleaved `Complex{T}` arrays are real tensors of shape (2, r, c) with strides (1, 2, 2*ld).
torch is used for device memory and streams only.
"""
from __future__ import annotations

import numpy as np

from .eltypes import ElType, from_torch


def cuarray(eltype: ElType, *shape, device="cuda"):
    """Uninitialised column-major array (Julia: CuArray{T}(undef, shape...))."""
    import torch
    shape = tuple(int(s) for s in (shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape))
    if eltype.is_complex:
        shape = (2, *shape)
    t = torch.empty(tuple(reversed(shape)), dtype=eltype.torch_dtype(), device=device)
    return t.permute(*reversed(range(len(shape))))


def to_cuarray(x: np.ndarray, eltype: ElType | None = None, device="cuda"):
    """Copies a numpy array to the device in column-major order.  Complex numpy arrays become
    interleaved (2, r, c) arrays of the real element type."""
    import torch
    x = np.asarray(x)
    if np.iscomplexobj(x):
        x = np.stack([x.real, x.imag], axis=0)
    t = torch.from_numpy(np.ascontiguousarray(x.transpose(*reversed(range(x.ndim)))))
    if eltype is not None:
        t = t.to(eltype.torch_dtype())
    t = t.to(device)
    return t.permute(*reversed(range(x.ndim)))


def to_numpy(t) -> np.ndarray:
    """Device array -> numpy array with the same logical shape (bfloat16 comes back as float32)."""
    import torch
    if t.dtype == torch.bfloat16:
        t = t.float()
    return t.detach().cpu().numpy()


def is_col_major(t) -> bool:
    if t.dim() == 1:
        return t.stride(0) == 1 or t.shape[0] <= 1
    return (t.stride(0) == 1 or t.shape[0] <= 1) and all(t.stride(i) >= 1 for i in range(1, t.dim()))


def leading_dimension(t, interleaved: bool = False) -> int:
    """Elements (pairs, for interleaved complex) between consecutive columns."""
    if interleaved:
        return max(t.stride(2) // 2, t.shape[1], 1) if t.dim() == 3 else 1
    if t.dim() == 1:
        return max(t.shape[0], 1)
    return max(t.stride(1), t.shape[0], 1) if t.shape[1] > 1 else max(t.shape[0], 1)


def eltype_of(t) -> ElType:
    return from_torch(t.dtype)
