"""matmul / matmatmul_ / mul_ — host mirror of src/matmul.jl over the C ABI.

`matmul` is the call site that replaces the reference's JIT compile + launch
(src/matmul.jl:38-43): it lowers a Config and device arrays to a gk_gemm_desc and calls gk_gemm
on the caller's current stream.  Nothing here computes; without the shared library the package
does not import.
"""
from __future__ import annotations

import ctypes as C
import threading

from . import _lib as L
from . import arrays
from . import cta_swizzle as CTASwizzle
from . import epilogue as Epilogue
from . import kernel as Kernel
from . import layout as Layout
from . import operator as Operator
from . import transform as Transform
from .config import Config, ConfigError, DimensionMismatch, get_config as _get_config, heuristic_block_shape
from .eltypes import BFloat16, ElType, Float16, Float32, promote_type

_handles: dict[int, C.c_void_p] = {}
_handles_lock = threading.Lock()


class GemmKernelsError(RuntimeError):
    pass


class DeviceTimeout(GemmKernelsError):
    """A bounded device-side wait gave up (GK_ERR_TIMEOUT); the CUDA context is still usable."""


def _raise(status: int):
    msg = L.last_error()
    if status == L.GK_ERR_INVALID_CONFIG:
        raise ConfigError(msg)
    if status == L.GK_ERR_DIMENSION_MISMATCH:
        raise DimensionMismatch(msg)
    if status == L.GK_ERR_UNSUPPORTED:
        raise Transform.UnsupportedFunctor(msg)
    if status == L.GK_ERR_TIMEOUT:
        raise DeviceTimeout(msg)
    raise GemmKernelsError(f"gk status {status}: {msg}")


def handle(device_index: int | None = None) -> C.c_void_p:
    """Per-device library handle (created on first use, kept for the life of the process)."""
    import torch
    if device_index is None:
        device_index = torch.cuda.current_device()
    with _handles_lock:
        h = _handles.get(device_index)
        if h is None:
            with torch.cuda.device(device_index):
                h = C.c_void_p()
                st = L.lib.gk_create(C.byref(h))
                if st != L.GK_OK:
                    _raise(st)
            _handles[device_index] = h
        return h


def poll_status(device_index: int | None = None) -> None:
    """Raises DeviceTimeout if a kernel launched on this device abandoned a wait."""
    code = C.c_int32(0)
    st = L.lib.gk_poll_status(handle(device_index), C.byref(code))
    if st != L.GK_OK:
        _raise(st)


# ------------------------------------------------------------------------------------------------
# lowering of the eight transform hooks (src/matmul.jl:8-15) to alpha / beta / activation
# ------------------------------------------------------------------------------------------------
def _functor(t):
    if t is None:
        return Transform.Identity()
    if isinstance(t, Transform.Elementwise):
        return t.f
    if isinstance(t, Transform.Functor):
        return t
    raise Transform.UnsupportedFunctor(f"expected Transform.Elementwise, got {t!r}")


def _fold_transforms(hooks: dict, has_bias: bool):
    """Net math of the reference: D = g_d( r_d( sum s_a(g_a(A)) s_b(g_b(B)) + s_c(g_c(C)) ) + bias ).
    Returns (alpha, beta, activation)."""
    alpha, beta, act = 1.0, 1.0, L.GK_ACT_NONE
    for name in ("global_to_shared_a", "shared_to_regs_a", "global_to_shared_b", "shared_to_regs_b"):
        f = _functor(hooks.get(name))
        if isinstance(f, Transform.Scale):
            alpha *= float(f.factor)
        elif not isinstance(f, (Transform.Identity, Transform.Cast)):
            raise Transform.UnsupportedFunctor(
                f"transform_{name} = {f!r}: operands go from TMA to the tensor cores without passing "
                "through registers, so only identity, Cast and Scale can be applied to A and B")
    for name in ("global_to_shared_c", "shared_to_regs_c"):
        f = _functor(hooks.get(name))
        if isinstance(f, Transform.Scale):
            beta *= float(f.factor)
        elif not isinstance(f, (Transform.Identity, Transform.Cast)):
            raise Transform.UnsupportedFunctor(f"transform_{name} = {f!r}: only identity, Cast and Scale apply to C")
    f = _functor(hooks.get("regs_to_shared_d"))
    if isinstance(f, Transform.Scale):
        alpha *= float(f.factor); beta *= float(f.factor)
    elif isinstance(f, (Transform.ReLU, Transform.GELU)):
        if has_bias:
            raise Transform.UnsupportedFunctor(
                "an activation in transform_regs_to_shared_d runs before the bias is added; the fused "
                "epilogue applies activations last — put it in transform_shared_to_global_d")
        act = L.GK_ACT_RELU if isinstance(f, Transform.ReLU) else L.GK_ACT_GELU
    elif not isinstance(f, (Transform.Identity, Transform.Cast)):
        raise Transform.UnsupportedFunctor(f"transform_regs_to_shared_d = {f!r}")
    f = _functor(hooks.get("shared_to_global_d"))
    if isinstance(f, Transform.Scale):
        if has_bias or act != L.GK_ACT_NONE:
            raise Transform.UnsupportedFunctor("Scale in transform_shared_to_global_d after a bias or activation is not fused")
        alpha *= float(f.factor); beta *= float(f.factor)
    elif isinstance(f, (Transform.ReLU, Transform.GELU)):
        if act != L.GK_ACT_NONE:
            raise Transform.UnsupportedFunctor("two activations requested")
        act = L.GK_ACT_RELU if isinstance(f, Transform.ReLU) else L.GK_ACT_GELU
    elif not isinstance(f, (Transform.Identity, Transform.Cast)):
        raise Transform.UnsupportedFunctor(f"transform_shared_to_global_d = {f!r}")
    return alpha, beta, act


def _compute_and_op(op):
    if isinstance(op, Operator.TCGen05Operator):
        name = getattr(op.CT, "name", "")
        comp = {"Float16": L.GK_F16, "BFloat16": L.GK_BF16, "TF32": L.GK_TF32, "Float32": L.GK_TF32}.get(name)
        if comp is None:
            raise ConfigError(f"TCGen05Operator cannot compute in {op.CT}")
        return L.GK_OP_TCGEN05, comp
    if isinstance(op, Operator.WMMAOp):
        name = getattr(op.CT, "name", "")
        comp = {"Float16": L.GK_F16, "BFloat16": L.GK_BF16}.get(name)
        if comp is None:
            raise ConfigError(f"WMMA operators compute in Float16, not {op.CT}")
        return L.GK_OP_TCGEN05, comp
    if isinstance(op, Operator.TropicalFPUOp):
        return L.GK_OP_FPU_TROPICAL, op.AT.gk
    if isinstance(op, Operator.FPUOp):
        return L.GK_OP_FPU, op.AT.gk
    raise ConfigError(f"unknown operator {op!r}")


_NUMBER = {"real": L.GK_REAL, "complex": L.GK_COMPLEX, "dual": L.GK_DUAL}


def lower(conf: Config, a, b, c, d, hooks: dict, epilogue, kernel):
    """Config + arrays -> (GemmDesc, EpilogueDesc, pointers).  Pure host logic."""
    M, N, K = (conf.matmul_shape[k] for k in "MNK")
    op, comp = _compute_and_op(conf.operator)
    number = _NUMBER[conf.operator.number]
    if kernel is Kernel.matmul_pipelined and conf.block_shape["K"] < 2 * conf.compute_op_shape["K"]:
        raise ConfigError("Need at least two stages to use a pipelined kernel, i.e. BLOCK_K ≥ 2 * OPERATOR_K")

    has_bias = isinstance(epilogue, Epilogue.Bias)
    alpha, beta, act = _fold_transforms(hooks, has_bias)

    la, lb, lc, ld_ = conf.global_a_layout, conf.global_b_layout, conf.global_c_layout, conf.global_d_layout
    desc = L.GemmDesc(number=number, m=M, n=N, k=K, compute=comp, op=op, alpha=alpha, beta=beta,
                      tile_n=conf.tile_n, cta_group=conf.cta_group, stages=conf.stages,
                      k_blocks_per_stage=conf.k_blocks_per_stage)
    desc.trans_a = 0 if la.col_major else 1
    desc.trans_b = 0 if lb.col_major else 1
    sw = conf.cta_swizzle
    if isinstance(sw, (CTASwizzle.HorizontallyTiled, CTASwizzle.VerticallyTiled)):
        desc.raster, desc.raster_group = sw.raster, sw.tile
    elif isinstance(sw, CTASwizzle.LebesgueCurve):
        desc.raster, desc.raster_group = sw.raster, conf.raster_group
    else:
        # Identity only fixes the order of block indices in the reference (it is the default of every
        # configuration); which tiles run together is up to the hardware scheduler there, so the
        # persistent scheduler keeps its own band raster.
        desc.raster, desc.raster_group = L.GK_RASTER_AUTO, conf.raster_group

    def operand(arr, layout, rows, cols, name):
        """-> (ptr, dtype, ld, plane, layout_kind)"""
        if layout.zero or arr is None:
            if arr is None and not layout.zero:
                raise GemmKernelsError(f"{name} is None but its layout is {layout!r}")
            et = layout.eltype
            return None, et.real.gk if et.is_complex else et.gk, max(rows, 1), 0, L.GK_LAYOUT_ZERO
        et = arrays.eltype_of(arr)
        want = layout.eltype.real if layout.eltype.is_complex else layout.eltype
        if et != want:
            raise ConfigError(f"{name} holds {et} but its layout is {layout!r}")
        if layout.diagonal:
            # the diagonal is the first M elements of the array's memory (the reference's harness
            # allocates a full M x K matrix and uses its first column, configs/configs.jl:338-340)
            if arr.numel() < rows or (arr.dim() >= 1 and arr.stride(0) != 1 and arr.shape[0] > 1):
                raise DimensionMismatch(f"{name}: Diagonal layout needs at least {rows} contiguous elements")
            return arr.data_ptr(), et.gk, max(rows, 1), 0, L.GK_LAYOUT_DIAGONAL
        if number != L.GK_REAL:
            if layout.split:
                if arr.dim() != 3 or arr.shape[2] != 2 or tuple(arr.shape[:2]) != (rows, cols):
                    raise DimensionMismatch(f"{name}: expected planar ({rows}, {cols}, 2), got {tuple(arr.shape)}")
                return arr.data_ptr(), et.gk, arrays.leading_dimension(arr), arr.stride(2), L.GK_LAYOUT_DENSE
            if arr.dim() != 3 or arr.shape[0] != 2 or tuple(arr.shape[1:]) != (rows, cols):
                raise DimensionMismatch(f"{name}: expected interleaved (2, {rows}, {cols}), got {tuple(arr.shape)}")
            return arr.data_ptr(), et.gk, arrays.leading_dimension(arr, True), 0, L.GK_LAYOUT_DENSE
        if arr.dim() != 2 or tuple(arr.shape) != (rows, cols):
            raise DimensionMismatch(f"Dimensions do not match: {name} is {tuple(arr.shape)}, expected ({rows}, {cols})")
        if not arrays.is_col_major(arr):
            raise GemmKernelsError(f"{name} must be stored column-major (stride 1 along its first dimension)")
        return arr.data_ptr(), et.gk, arrays.leading_dimension(arr), 0, L.GK_LAYOUT_DENSE

    a_rows, a_cols = (M, K) if la.col_major else (K, M)
    b_rows, b_cols = (K, N) if lb.col_major else (N, K)
    if la.diagonal:
        a_ptr, desc.dtype_a, desc.lda, desc.plane_a, desc.layout_a = operand(a, la, M, 1, "A")
    else:
        a_ptr, desc.dtype_a, desc.lda, desc.plane_a, desc.layout_a = operand(a, la, a_rows, a_cols, "A")
    b_ptr, desc.dtype_b, desc.ldb, desc.plane_b, desc.layout_b = operand(b, lb, b_rows, b_cols, "B")
    c_ptr, desc.dtype_c, desc.ldc, desc.plane_c, desc.layout_c = operand(c, lc, M, N, "C")
    d_ptr, desc.dtype_d, desc.ldd, desc.plane_d, _ = operand(d, ld_, M, N, "D")
    if desc.layout_c == L.GK_LAYOUT_ZERO:
        desc.dtype_c, desc.ldc = desc.dtype_d, desc.ldd
        desc.beta = 0.0

    epi = L.EpilogueDesc(activation=act)
    if has_bias:
        bias = epilogue.bias
        ptr = bias if isinstance(bias, int) else bias.data_ptr()
        if not isinstance(bias, int):
            import torch
            if bias.dtype != torch.float32:
                raise Transform.UnsupportedFunctor("Epilogue.Bias takes a Float32 bias (src/epilogue.jl:40)")
            need = M if epilogue.axis == "row" else N
            if bias.numel() != need:
                raise DimensionMismatch(f"bias has {bias.numel()} elements, expected {need}")
        epi.bias = ptr
        epi.bias_axis = L.GK_BIAS_ROW if epilogue.axis == "row" else L.GK_BIAS_COL
    elif not isinstance(epilogue, Epilogue.Default):
        raise Transform.UnsupportedFunctor(f"epilogue {epilogue!r} is not Epilogue.Default or Epilogue.Bias")
    return desc, epi, (a_ptr, b_ptr, c_ptr, d_ptr)


def _wants_workspace(desc) -> bool:
    """Cases in which the library can use a workspace: interleaved complex / dual operands (split into
    planes first), real tensor-core products with few output tiles and a long K (split-K), and FFMA
    products (the tiles of a partly filled last round, or of a grid too small for the GPU, are cut along K)."""
    if desc.number != L.GK_REAL:
        return desc.plane_a == 0 or desc.plane_b == 0
    if desc.op == L.GK_OP_FPU and desc.dtype_d == L.GK_F32:
        if desc.m * desc.n <= 148 * 128 * 128:                      # too few tiles to fill the GPU: all cut along K
            return desc.k >= 256
        return desc.m * desc.n >= (1 << 22) and desc.k >= 1024      # the FFMA kernel's tail split
    return desc.m * desc.n <= (1 << 22) and desc.k >= 2048


# Scratch buffers the package lends to gk_gemm when the caller passes none: one per (device, stream),
# allocated on first need, replaced only by a larger one, never per call.  Kernels that use a buffer
# are ordered by the stream it belongs to, so successive calls on that stream may share it.
_workspaces: dict = {}
_workspaces_lock = threading.Lock()


def _workspace_bytes(ws) -> int:
    return 0 if ws is None else ws.numel() * ws.element_size()


def _check_user_workspace(h, desc, epi, workspace):
    """A workspace the caller supplies must cover what gk_gemm_query reports when the library cannot
    do without it (interleaved operands); for the optional uses the library itself falls back."""
    import torch
    if desc.number != L.GK_REAL and (desc.plane_a == 0 or desc.plane_b == 0):
        plan = L.GemmPlan()
        st = L.lib.gk_gemm_query(h, C.byref(desc), C.byref(epi), C.byref(plan))
        if st != L.GK_OK:
            _raise(st)
        if _workspace_bytes(workspace) < plan.workspace_bytes:
            raise GemmKernelsError(f"workspace holds {_workspace_bytes(workspace)} bytes, this product needs {plan.workspace_bytes}")
    if workspace.data_ptr() % 256:
        raise GemmKernelsError("workspace must be 256-byte aligned")


def lend_workspace(device, stream: int, nbytes: int):
    """The lent scratch buffer of (device, stream), at least `nbytes` long: allocated on first need,
    replaced only by a larger one (never per call)."""
    import torch
    key = (device.index, int(stream))
    with _workspaces_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            size = max(nbytes, 2 * (ws.numel() if ws is not None else 0))
            # allocate under the caller's stream so the caching allocator ties the block to it
            if int(stream) == torch.cuda.current_stream(device).cuda_stream:
                ws = torch.empty(size, dtype=torch.uint8, device=device)
            else:
                with torch.cuda.stream(torch.cuda.ExternalStream(int(stream), device=device)):
                    ws = torch.empty(size, dtype=torch.uint8, device=device)
            _workspaces[key] = ws
    return ws


def _auto_workspace(h, desc, epi, like, stream: int):
    """The lent workspace of (device, stream), grown to the size gk_gemm_query reports, or None."""
    plan = L.GemmPlan()
    st = L.lib.gk_gemm_query(h, C.byref(desc), C.byref(epi), C.byref(plan))
    if st != L.GK_OK:
        _raise(st)
    if not plan.workspace_bytes:
        return None
    return lend_workspace(like.device, stream, plan.workspace_bytes)


def matmul(conf: Config, a, b, c, d, *,
           transform_global_to_shared_a=None, transform_global_to_shared_b=None,
           transform_global_to_shared_c=None, transform_shared_to_global_d=None,
           transform_shared_to_regs_a=None, transform_shared_to_regs_b=None,
           transform_shared_to_regs_c=None, transform_regs_to_shared_d=None,
           epilogue=None, kernel=Kernel.matmul_singlestage, stream=None, workspace=None):
    """GemmKernels.matmul(conf, a, b, c, d; ...) (src/matmul.jl:7-44): D = epilogue(A*B + C),
    enqueued asynchronously on the current CUDA stream.  Raises ConfigError for combinations the
    engine cannot run (the reference's tests count that as "skipped")."""
    import torch
    hooks = {
        "global_to_shared_a": transform_global_to_shared_a, "global_to_shared_b": transform_global_to_shared_b,
        "global_to_shared_c": transform_global_to_shared_c, "shared_to_global_d": transform_shared_to_global_d,
        "shared_to_regs_a": transform_shared_to_regs_a, "shared_to_regs_b": transform_shared_to_regs_b,
        "shared_to_regs_c": transform_shared_to_regs_c, "regs_to_shared_d": transform_regs_to_shared_d,
    }
    desc, epi, (pa, pb, pc, pd) = lower(conf, a, b, c, d, hooks, epilogue or Epilogue.Default(), kernel)
    dev = d.device.index if d.device.index is not None else torch.cuda.current_device()
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        if workspace is not None:
            _check_user_workspace(handle(dev), desc, epi, workspace)
        elif _wants_workspace(desc):
            workspace = _auto_workspace(handle(dev), desc, epi, d, s)
        ws = workspace.data_ptr() if workspace is not None else None
        st = L.lib.gk_gemm(handle(dev), C.byref(desc), pa, pb, pc, pd, C.byref(epi), ws, _workspace_bytes(workspace),
                           C.c_void_p(s))
    if st != L.GK_OK:
        _raise(st)
    return None


def matmul_batched(conf: Config, a, b, c, d, *, epilogue=None, kernel=Kernel.matmul_singlestage, stream=None,
                   **transforms):
    """`batch` independent products of one shape in one launch: D[:, :, i] = epilogue(A[:, :, i] * B[:, :, i]
    + C[:, :, i]).  `d` is a 3-D column-major array (M, N, batch); `a`, `b` and `c` are 3-D with the same
    last extent, or 2-D to share one matrix between all products (`c` may be None).  `conf` describes
    one product.  The reference has no batched entry point; on the tensor-core path the persistent
    scheduler walks (product, tile) pairs, so small products fill the GPU together."""
    import torch
    if d.dim() != 3:
        raise DimensionMismatch("matmul_batched: D must be (M, N, batch)")
    nb = d.shape[2]
    if nb == 0:
        return None

    def first(x, name):
        if x is None or x.dim() == 2:
            return x, 0
        if x.dim() != 3 or x.shape[2] != nb:
            raise DimensionMismatch(f"matmul_batched: {name} has shape {tuple(x.shape)}, expected a last extent of {nb}")
        return x[:, :, 0], (x.stride(2) if nb > 1 else 0)

    (a0, sa), (b0, sb), (c0, sc), (d0, sd) = first(a, "A"), first(b, "B"), first(c, "C"), first(d, "D")
    hooks = {k.replace("transform_", ""): v for k, v in transforms.items()}
    desc, epi, (pa, pb, pc, pd) = lower(conf, a0, b0, c0, d0, hooks, epilogue or Epilogue.Default(), kernel)
    desc.batch = nb
    desc.batch_stride_a, desc.batch_stride_b, desc.batch_stride_c, desc.batch_stride_d = sa, sb, sc, sd
    dev = d.device.index if d.device.index is not None else torch.cuda.current_device()
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        st = L.lib.gk_gemm(handle(dev), C.byref(desc), pa, pb, pc, pd, C.byref(epi), None, 0, C.c_void_p(s))
    if st != L.GK_OK:
        _raise(st)
    return None


class BoundMatmul:
    """`matmul` with its arguments lowered once: calling the object enqueues the same GEMM again
    (same arrays, same descriptors) for the cost of one FFI call.  The Julia package gets the same
    effect from its compiled-kernel cache; in Python the per-call lowering (~25 us) would otherwise
    dominate small problems.  The arrays are kept alive by the object."""

    def __init__(self, conf, a, b, c, d, hooks, epilogue, kernel, workspace):
        import torch
        self._keep = (a, b, c, d, epilogue, workspace)
        self.desc, self.epi, self.ptrs = lower(conf, a, b, c, d, hooks, epilogue, kernel)
        self.device = d.device.index if d.device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(self.device):
            self.handle = handle(self.device)
            if workspace is not None:
                _check_user_workspace(self.handle, self.desc, self.epi, workspace)
            elif _wants_workspace(self.desc):
                # a bound product owns its scratch: it may be replayed on any stream
                plan = L.GemmPlan()
                st = L.lib.gk_gemm_query(self.handle, C.byref(self.desc), C.byref(self.epi), C.byref(plan))
                if st != L.GK_OK:
                    _raise(st)
                if plan.workspace_bytes:
                    workspace = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device=d.device)
                    self._keep += (workspace,)
        self.ws = workspace.data_ptr() if workspace is not None else None
        self.ws_bytes = _workspace_bytes(workspace)
        self._torch = torch

    def __call__(self, stream=None):
        """Enqueues on `stream` (a raw CUDA stream handle) or on torch's current stream of the
        device that holds D; that device must be current."""
        s = stream if stream is not None else self._torch.cuda.current_stream(self.device).cuda_stream
        pa, pb, pc, pd = self.ptrs
        st = L.lib.gk_gemm(self.handle, C.byref(self.desc), pa, pb, pc, pd, C.byref(self.epi), self.ws, self.ws_bytes,
                           C.c_void_p(s))
        if st != L.GK_OK:
            _raise(st)


def bind(conf: Config, a, b, c, d, *, epilogue=None, kernel=Kernel.matmul_singlestage, workspace=None, **transforms):
    """Lower `matmul(conf, a, b, c, d; ...)` once and return a callable that enqueues it."""
    hooks = {k.replace("transform_", ""): v for k, v in transforms.items()}
    return BoundMatmul(conf, a, b, c, d, hooks, epilogue or Epilogue.Default(), kernel, workspace)


def matmul_host(conf: Config, a, b, c, d, *, epilogue=None, kernel=Kernel.matmul_singlestage, stream=None,
                device_index=None, a_on_device=False, **transforms):
    """`matmul` for matrices in host memory (column-major CPU tensors, ideally pinned): copies the
    operands to the device, runs the GEMM and copies D back into `d`; returns when `d` is complete.
    With `a_on_device=True`, `a` is a device array that is used where it is (the sharded path: A is
    uploaded by one rank and broadcast over NVLink, every rank uploads only its block of B).
    Julia counterpart: calling the shim's `matmul` with `Array`s instead of `CuArray`s."""
    import torch
    hooks = {k.replace("transform_", ""): v for k, v in transforms.items()}
    epilogue = epilogue or Epilogue.Default()
    desc, epi, (pa, pb, pc, pd) = lower(conf, a, b, c, d, hooks, epilogue, kernel)
    if a_on_device:
        desc.a_resident = 1            # A is a device array already (resident or just broadcast): used in place
    dev = device_index if device_index is not None else torch.cuda.current_device()
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        st = L.lib.gk_gemm_host(handle(dev), C.byref(desc), pa, pb, pc, pd, C.byref(epi), C.c_void_p(s))
    if st != L.GK_OK:
        _raise(st)
    return None


def query(conf: Config, a, b, c, d, *, epilogue=None, kernel=Kernel.matmul_singlestage, **hooks) -> L.GemmPlan:
    """What `matmul` would launch for these arguments (kernel family, grid, shared memory, TMEM
    columns); launches nothing.  This is where the reference checked its shared-memory and thread
    limits (src/matmul.jl:24-41)."""
    import torch
    hooks = {k.replace("transform_", ""): v for k, v in hooks.items()}
    desc, epi, _ = lower(conf, a, b, c, d, hooks, epilogue or Epilogue.Default(), kernel)
    plan = L.GemmPlan()
    st = L.lib.gk_gemm_query(handle(), C.byref(desc), C.byref(epi), C.byref(plan))
    if st != L.GK_OK:
        _raise(st)
    return plan


# ------------------------------------------------------------------------------------------------
# BLAS-like front end (src/matmul.jl:47-215)
# ------------------------------------------------------------------------------------------------
_config_cache: dict = {}
_config_lock = threading.Lock()

# (compute type, compute type, eltype(C)) triples that go to the tensor cores by default.  The
# reference lists the two Float16 rows (src/matmul.jl:85-89); BFloat16 is the B200 addition.
_TENSOR_TYPES = {("Float16", "Float16", "Float16"), ("Float16", "Float16", "Float32"),
                 ("BFloat16", "BFloat16", "BFloat16"), ("BFloat16", "BFloat16", "Float32")}


def create_config(A: ElType, sizeA, stridesA, transA: bool, B: ElType, sizeB, stridesB, transB: bool,
                  Ct: ElType, sizeC, stridesC, zero_alpha: bool, zero_beta: bool, wmma):
    """create_config of src/matmul.jl:66-183."""
    m = sizeA[1] if transA else sizeA[0]
    k = sizeA[0] if transA else sizeA[1]
    n = sizeB[0] if transB else sizeB[1]
    if m != sizeC[0] or n != sizeC[1] or k != (sizeB[1] if transB else sizeB[0]):
        raise DimensionMismatch("Dimensions do not match")
    a_base = Layout.RowMajor if transA else Layout.ColMajor
    b_base = Layout.RowMajor if transB else Layout.ColMajor
    a_al = Layout.UnsafeAlignedRowMajor if transA else Layout.UnsafeAlignedColMajor
    b_al = Layout.UnsafeAlignedRowMajor if transB else Layout.UnsafeAlignedColMajor
    ct = promote_type(A, B)
    use_tensor = wmma if wmma is not None else ((ct.name, ct.name, Ct.name) in _TENSOR_TYPES)
    if use_tensor:
        shared_a, shared_b = Layout.Padded(a_al(ct), 8), Layout.Padded(b_al(ct), 8)
    else:
        shared_a, shared_b = Layout.Padded(a_al(A), 8), Layout.Padded(b_al(B), 8)
    shared_c = Layout.Zero(Ct) if zero_beta else Layout.UnsafeAlignedColMajor(Ct)
    shared_d = Layout.UnsafeAlignedColMajor(Ct)
    block_shape = heuristic_block_shape(shared_a, shared_b, shared_c, shared_d) if use_tensor \
        else {"M": 128, "N": 128, "K": 32}
    a_aligned = (stridesA[1] * A.size) % 16 == 0
    b_aligned = (stridesB[1] * B.size) % 16 == 0
    c_aligned = (stridesC[1] * Ct.size) % 16 == 0
    if zero_alpha:
        ga, gb = Layout.Zero(A), Layout.Zero(B)
    else:
        ga = a_al(A) if a_aligned and m % block_shape["M"] == 0 and k % block_shape["K"] == 0 else a_base(A)
        gb = b_al(B) if b_aligned and k % block_shape["K"] == 0 and n % block_shape["N"] == 0 else b_base(B)
    cd_ok = c_aligned and m % block_shape["M"] == 0 and n % block_shape["N"] == 0
    gc = Layout.Zero(Ct) if zero_beta else (Layout.UnsafeAlignedColMajor(Ct) if cd_ok else Layout.ColMajor(Ct))
    gd = Layout.UnsafeAlignedColMajor(Ct) if cd_ok else Layout.ColMajor(Ct)
    if use_tensor:
        comp = Operator.TF32 if ct.name == "Float32" else ct
        op = Operator.TCGen05Operator(comp, Ct)
    else:
        op = Operator.FPUOp(8, 8, 1, 4, 8, 1, ct, Ct)
    conf = _get_config(gemm_shape=(m, n, k), block_shape=block_shape, operator=op,
                       global_a_layout=ga, global_b_layout=gb, global_c_layout=gc, global_d_layout=gd,
                       shared_a_layout=shared_a, shared_b_layout=shared_b, shared_c_layout=shared_c,
                       shared_d_layout=shared_d, is_a_col_major=not transA, is_b_col_major=not transB)
    both_aligned = ga.aligned and gb.aligned and not ga.zero
    return conf, ct, (Kernel.matmul_pipelined if both_aligned else Kernel.matmul_singlestage)


def get_config_cached(*args):
    """The memo cache of src/matmul.jl:58-65."""
    with _config_lock:
        val = _config_cache.get(args)
    if val is None:
        val = create_config(*args)
        with _config_lock:
            _config_cache[args] = val
    return val


def matmatmul_(Cm, transA: str, transB: str, A, B, alpha, beta, *, wmma=None):
    """GemmKernels.matmatmul!(C, transA, transB, A, B, alpha, beta; wmma) (src/matmul.jl:185-204).
    C = alpha * op(A) * op(B) + beta * C in place; returns C."""
    def strides(t):
        return (t.stride(0), arrays.leading_dimension(t))
    conf, compute_type, kernel = get_config_cached(
        arrays.eltype_of(A), tuple(A.shape), strides(A), transA == "T",
        arrays.eltype_of(B), tuple(B.shape), strides(B), transB == "T",
        arrays.eltype_of(Cm), tuple(Cm.shape), strides(Cm),
        alpha == 0, beta == 0, wmma)
    matmul(conf, A, B, Cm, Cm,
           transform_shared_to_regs_a=Transform.Elementwise(Transform.Scale(alpha)),
           transform_shared_to_regs_c=Transform.Elementwise(Transform.Scale(beta)),
           kernel=kernel)
    return Cm


def mul_(Cm, A, B, alpha=True, beta=False):
    """GemmKernels.mul!(C, A, B, alpha, beta) (src/matmul.jl:207-215).  A transposed operand is a
    row-major view of its parent (what `parent.T` gives in torch), mirroring Julia's
    Transpose/Adjoint wrappers."""
    def unwrap(X):
        if arrays.is_col_major(X):
            return "N", X
        if X.dim() == 2 and X.stride(1) == 1:
            return "T", X.T
        raise GemmKernelsError("operand is neither column-major nor the transpose of a column-major array")
    ta, Ap = unwrap(A)
    tb, Bp = unwrap(B)
    return matmatmul_(Cm, ta, tb, Ap, Bp, float(alpha), float(beta))
