"""Tensor contraction entry point: `contract_(D, modes_d, A, modes_a, B, modes_b, alpha, beta, C)`.

The reference ships no contraction function; its benchmark
(benchmarks/tensor-contractions/run.jl:88-131) expresses one contraction through custom Layouts.
This is the entry point the engine defines for it (Julia: `GemmKernels.contract!`): mode strings as
in the TCCG benchmark notation, tensors read in place with their own strides.
"""
from __future__ import annotations

import ctypes as C

from . import _lib as L
from . import arrays
from .matmul import _raise, handle
from .operator import TF32


def _desc(D, modes_d, A, modes_a, B, modes_b, alpha, beta, Cin, compute, force_gather, tile_n, cta_group):
    for name, t, modes in (("A", A, modes_a), ("B", B, modes_b), ("D", D, modes_d)):
        if t.dim() != len(modes):
            raise ValueError(f"{name} has {t.dim()} dimensions but {len(modes)} modes ('{modes}')")
        if len(modes) > L.GK_MAX_MODES:
            raise ValueError(f"at most {L.GK_MAX_MODES} modes per tensor")
    d = L.ContractDesc(rank_a=len(modes_a), rank_b=len(modes_b), rank_c=len(modes_d), alpha=float(alpha),
                       beta=float(beta), force_gather=int(force_gather), tile_n=tile_n, cta_group=cta_group)
    for i, ch in enumerate(modes_a):
        d.modes_a[i], d.extents_a[i], d.strides_a[i] = ord(ch), A.shape[i], A.stride(i)
    for i, ch in enumerate(modes_b):
        d.modes_b[i], d.extents_b[i], d.strides_b[i] = ord(ch), B.shape[i], B.stride(i)
    csrc = Cin if Cin is not None else D
    for i, ch in enumerate(modes_d):
        d.modes_c[i], d.extents_c[i] = ord(ch), D.shape[i]
        d.strides_d[i], d.strides_c[i] = D.stride(i), csrc.stride(i)
    ea, eb, ed = arrays.eltype_of(A), arrays.eltype_of(B), arrays.eltype_of(D)
    d.dtype_a, d.dtype_b, d.dtype_d = ea.gk, eb.gk, ed.gk
    d.dtype_c = arrays.eltype_of(csrc).gk
    if compute is None:
        compute = {"Float16": L.GK_F16, "BFloat16": L.GK_BF16}.get(ea.name, L.GK_F32)
    elif compute is TF32:
        compute = L.GK_TF32
    elif not isinstance(compute, int):
        compute = compute.gk
    d.compute = compute
    return d


def contract_query(D, modes_d, A, modes_a, B, modes_b, alpha=1.0, beta=0.0, C_in=None, *, compute=None,
                   force_gather=False, tile_n=0, cta_group=0) -> L.GemmPlan:
    """Which kernel `contract_` would use and how much workspace it needs."""
    d = _desc(D, modes_d, A, modes_a, B, modes_b, alpha, beta, C_in, compute, force_gather, tile_n, cta_group)
    plan = L.GemmPlan()
    st = L.lib.gk_contract_query(handle(), C.byref(d), C.byref(plan))
    if st != L.GK_OK:
        _raise(st)
    return plan


def contract_(D, modes_d: str, A, modes_a: str, B, modes_b: str, alpha=1.0, beta=0.0, C_in=None, *,
              compute=None, workspace=None, force_gather=False, tile_n=0, cta_group=0, stream=None):
    """D[modes_d] = alpha * sum over shared modes of A[modes_a] * B[modes_b] + beta * C[modes_d].

    Tensors are torch CUDA tensors with any strides (Julia arrays are column-major: use `cuarray`).
    C defaults to D (in place) when beta != 0.  A mode in A, B and D is a batch mode: one contraction
    per index value.  If the contraction can use scratch memory (offset tables of the gather kernel,
    partial sums of a split along K) and no `workspace` (uint8/int64 CUDA tensor) is given, the
    package lends its grow-only buffer of this device and stream.  Returns D."""
    import torch
    if beta != 0 and C_in is None:
        C_in = D
    d = _desc(D, modes_d, A, modes_a, B, modes_b, alpha, beta, C_in, compute, force_gather, tile_n, cta_group)
    dev = D.device.index if D.device.index is not None else torch.cuda.current_device()
    ws_ptr, ws_bytes = None, 0
    with torch.cuda.device(dev):
        h = handle(dev)
        s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
        if workspace is None:
            plan = L.GemmPlan()
            st = L.lib.gk_contract_query(h, C.byref(d), C.byref(plan))
            if st != L.GK_OK:
                _raise(st)
            if plan.workspace_bytes:
                from .matmul import lend_workspace
                workspace = lend_workspace(D.device, s, plan.workspace_bytes)
        if workspace is not None:
            ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
        st = L.lib.gk_contract(h, C.byref(d), A.data_ptr(), B.data_ptr(), C_in.data_ptr() if C_in is not None else None,
                               D.data_ptr(), ws_ptr, ws_bytes, C.c_void_p(s))
    if st != L.GK_OK:
        _raise(st)
    return D


class BoundContraction:
    """`contract_` with its descriptor built once (and its workspace allocated once): calling the
    object enqueues the same contraction again for the cost of one FFI call."""

    def __init__(self, D, modes_d, A, modes_a, B, modes_b, alpha=1.0, beta=0.0, C_in=None, *, compute=None,
                 workspace=None, force_gather=False, tile_n=0, cta_group=0):
        import torch
        if beta != 0 and C_in is None:
            C_in = D
        self.desc = _desc(D, modes_d, A, modes_a, B, modes_b, alpha, beta, C_in, compute, force_gather, tile_n, cta_group)
        self.device = D.device.index if D.device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(self.device):
            self.handle = handle(self.device)
            if workspace is None:
                plan = L.GemmPlan()
                st = L.lib.gk_contract_query(self.handle, C.byref(self.desc), C.byref(plan))
                if st != L.GK_OK:
                    _raise(st)
                if plan.workspace_bytes:
                    workspace = torch.empty(plan.workspace_bytes // 8 + 1, dtype=torch.int64, device=D.device)
        self.ws = (workspace.data_ptr(), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
        self.ptrs = (A.data_ptr(), B.data_ptr(), C_in.data_ptr() if C_in is not None else None, D.data_ptr())
        self._keep = (A, B, C_in, D, workspace)
        self._torch = torch

    def __call__(self, stream=None):
        s = stream if stream is not None else self._torch.cuda.current_stream(self.device).cuda_stream
        st = L.lib.gk_contract(self.handle, C.byref(self.desc), *self.ptrs, *self.ws, C.c_void_p(s))
        if st != L.GK_OK:
            _raise(st)


def bind_contract(*args, **kwargs) -> BoundContraction:
    """Same arguments as `contract_` (without `stream`); returns a callable that enqueues it."""
    return BoundContraction(*args, **kwargs)
