"""The reference's configuration list (configs/configs.jl:492-690) as library code: every entry has the
reference's name, builds its `Config`, draws inputs on the device, and knows how to run itself and its
cuBLAS baseline.  Used by the benchmark runner; the parity tests build the same configurations on their
own so that a slip here cannot hide a slip there.

Differences from the reference list: the "WMMA GEMM parameters" sweep over warp layouts
(configs.jl:604-621) describes how warps of a CUDA-core-era CTA split a tile and has no effect on the
tcgen05 engine, so one entry per (block shape, kernel, zero_c) is kept instead of one per warp layout.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable

from . import eltypes as T
from . import epilogue as Epilogue
from . import kernel as Kernel
from . import layout as Layout
from . import operator as Operator
from . import transform as Transform
from .config import Config, ConfigError, get_config


def _tt(ta, tb):
    return ("T" if ta else "N") + ("T" if tb else "N")


@dataclass
class Configuration:
    """One benchmark / test case (configs.jl:13-33)."""
    name: str
    config: Config
    shapes: dict                      # operand name -> shape of the array to allocate
    eltypes: dict                     # operand name -> ElType
    kwargs: Callable[[dict], dict] = field(default=lambda ops: {})   # extra arguments of matmul (epilogue, transforms)
    baseline: Callable[[dict], None] | None = None                   # cuBLAS product of the same operands, or None
    kernel: object = Kernel.matmul_singlestage

    @property
    def flops(self) -> float:
        s = self.config.matmul_shape
        return 2.0 * s["M"] * s["N"] * s["K"]

    def generate_inputs(self, seed: int = 0) -> dict:
        """Device operands in column-major order, values uniform in [0, 1) (integers: 0..3)."""
        import torch
        from . import arrays
        g = torch.Generator(device="cuda").manual_seed(seed)
        ops = {}
        for k, shape in self.shapes.items():
            et = self.eltypes[k]
            t = arrays.cuarray(et, *shape)
            if k != "d":
                r = torch.rand(tuple(reversed(t.shape)), device="cuda", generator=g)
                if et.name.startswith("Int"):
                    r = (r * 4).floor()
                t.copy_(r.permute(*reversed(range(r.dim()))))
            ops[k] = t
        return ops

    def bind(self, ops: dict):
        from .matmul import bind
        return bind(self.config, ops["a"], ops["b"], ops.get("c"), ops["d"], kernel=self.kernel, **self.kwargs(ops))


def _layouts(et, ta, tb, aligned=True):
    col, row = (Layout.UnsafeAlignedColMajor, Layout.UnsafeAlignedRowMajor) if aligned else (Layout.ColMajor, Layout.RowMajor)
    return (row if ta else col)[et], (row if tb else col)[et]


def _plain_baseline(ta, tb):
    """cuBLAS through torch on the same device arrays: op(A) op(B) in the operands' type (the reference's
    baseline is `mul!` = cuBLAS gemmEx, configs.jl:87-93; the C addend is left out here, it does not
    change which library kernel runs)."""
    def run(ops):
        import torch
        torch.matmul(ops["a"].t() if ta else ops["a"], ops["b"].t() if tb else ops["b"])
    return run


def fpu_config(A, B, CD, ta, tb, op, block, M, N, K, tropical=False) -> Configuration:
    """@get_fpu_config / @get_tropical_config (configs.jl:163-222)."""
    om, on, ok, mb, nb, kb = op
    opcls = Operator.TropicalFPUOp if tropical else Operator.FPUOp
    la, lb = _layouts(A, ta, tb)
    if B is not A:
        lb = _layouts(B, ta, tb)[1]
    conf = get_config(gemm_shape=(M, N, K), block_shape=block, operator=opcls[om, on, ok, mb, nb, kb, A, CD],
                      global_a_layout=la, global_b_layout=lb, global_c_layout=Layout.UnsafeAlignedColMajor[CD],
                      global_d_layout=Layout.UnsafeAlignedColMajor[CD], is_a_col_major=not ta, is_b_col_major=not tb)
    kind = "Tropical GEMM" if tropical else "FPU GEMM"
    name = (f"{kind} {A}*{B}={CD} ({M}×{K}) · ({K}×{N}) ({_tt(ta, tb)}) OP ({om}, {on}, {ok}), "
            f"base shape ({mb}, {nb}, {kb})")
    base = None if tropical or A.name.startswith("Int") or A is not CD else _plain_baseline(ta, tb)
    return Configuration(name, conf, {"a": (K, M) if ta else (M, K), "b": (N, K) if tb else (K, N), "c": (M, N), "d": (M, N)},
                         {"a": A, "b": B, "c": CD, "d": CD}, baseline=base)


def wmma_config(AB, CD, ta, tb, block, op, M, N, K, zero_c=False, kernel=Kernel.matmul_pipelined, warps=(4, 2)) -> Configuration:
    """@get_wmma_config (configs.jl:224-266): block shape, warp grid (warps_per_block = WARPS_M * WARPS_N,
    compute_warp = block / warps) and operator shape all go to get_config, which raises ConfigError for the
    combinations its rules exclude."""
    la, lb = _layouts(AB, ta, tb)
    conf = get_config(gemm_shape=(M, N, K), block_shape=block, operator=Operator.WMMAOp[op[0], op[1], op[2], AB, CD],
                      warps_per_block=warps[0] * warps[1],
                      compute_warp=(block[0] // warps[0], block[1] // warps[1], op[2]),
                      global_a_layout=la, global_b_layout=lb,
                      global_c_layout=(Layout.Zero if zero_c else Layout.UnsafeAlignedColMajor)[CD],
                      global_d_layout=Layout.UnsafeAlignedColMajor[CD], is_a_col_major=not ta, is_b_col_major=not tb)
    name = (f"WMMA GEMM {AB}*{AB}{'' if zero_c else f'+{CD}'}={CD} ({M}×{K}) · ({K}×{N}) ({_tt(ta, tb)}) "
            f"Block ({block[0]}, {block[1]}, {block[2]}) Warps ({warps[0]}, {warps[1]}) OP ({op[0]}, {op[1]}, {op[2]})")
    if kernel is Kernel.matmul_singlestage:
        name += " singlestage"
    shapes = {"a": (K, M) if ta else (M, K), "b": (N, K) if tb else (K, N), "d": (M, N)}
    if not zero_c:
        shapes["c"] = (M, N)
    return Configuration(name, conf, shapes, {"a": AB, "b": AB, "c": CD, "d": CD},
                         baseline=_plain_baseline(ta, tb), kernel=kernel)


def wmma_bias_config(AB, CD, ta, tb, op, M, N, K) -> Configuration:
    """@get_wmma_bias_config (configs.jl:268-311): D = A*B + C + bias[n]."""
    la, lb = _layouts(AB, ta, tb)
    conf = get_config(gemm_shape=(M, N, K), operator=Operator.WMMAOp[op[0], op[1], op[2], AB, CD],
                      global_a_layout=la, global_b_layout=lb, global_c_layout=Layout.UnsafeAlignedColMajor[CD],
                      global_d_layout=Layout.UnsafeAlignedColMajor[CD], is_a_col_major=not ta, is_b_col_major=not tb)
    name = f"WMMA GEMM+bias {AB}*{AB}+{CD}={CD} ({M}×{K}) · ({K}×{N}) ({_tt(ta, tb)}) OP ({op[0]}, {op[1]}, {op[2]})"
    return Configuration(name, conf, {"a": (K, M) if ta else (M, K), "b": (N, K) if tb else (K, N), "c": (M, N),
                                      "d": (M, N), "bias": (N,)},
                         {"a": AB, "b": AB, "c": CD, "d": CD, "bias": T.Float32},
                         kwargs=lambda ops: {"epilogue": Epilogue.Bias(ops["bias"])}, baseline=_plain_baseline(ta, tb))


def wmma_diagonal_config(AB, CD, tb, op, M, N, K) -> Configuration:
    """@get_wmma_diagonal_config (configs.jl:313-383): A is the diagonal, stored as the first column."""
    lb = _layouts(AB, False, tb)[1]
    conf = get_config(gemm_shape=(M, N, K), operator=Operator.WMMAOp[op[0], op[1], op[2], AB, CD],
                      global_a_layout=Layout.Diagonal[AB], global_b_layout=lb,
                      global_c_layout=Layout.UnsafeAlignedColMajor[CD], global_d_layout=Layout.UnsafeAlignedColMajor[CD],
                      shared_a_layout=Layout.Padded[Layout.UnsafeAlignedColMajor[AB], 8], is_b_col_major=not tb)
    name = f"WMMA diagonal GEMM diag({AB})*{AB}={CD} ({M}×{K}) · ({K}×{N}) ({_tt(False, tb)}) OP ({op[0]}, {op[1]}, {op[2]})"
    return Configuration(name, conf, {"a": (M, K), "b": (N, K) if tb else (K, N), "c": (M, N), "d": (M, N)},
                         {"a": AB, "b": AB, "c": CD, "d": CD})


def wmma_complex_config(AB, CD, ta, tb, op, M, N, K, dual=False) -> Configuration:
    """@get_wmma_complex_config / @get_wmma_dual_config (configs.jl:385-490): interleaved Complex{T} /
    dual operands, C = 0."""
    opcls = Operator.WMMADualOp if dual else Operator.WMMAComplexOp
    cab = T.ComplexF16 if AB is T.Float16 else T.ComplexF32
    ccd = T.ComplexF32
    il = lambda t: (Layout.InterleavedRowMajor if t else Layout.InterleavedColMajor)
    conf = get_config(gemm_shape=(M, N, K), block_shape=(64, 64, 32), operator=opcls[op[0], op[1], op[2], AB, CD],
                      global_a_layout=il(ta)[cab], global_b_layout=il(tb)[cab],
                      global_c_layout=Layout.Zero[ccd], global_d_layout=Layout.InterleavedColMajor[ccd],
                      is_a_col_major=not ta, is_b_col_major=not tb)
    kind = f"WMMA Dual GEMM d{AB}*d{AB}=d{CD}" if dual else f"WMMA Complex GEMM {AB}*{AB}={CD}"
    name = f"{kind} ({M}×{K}) · ({K}×{N}) ({_tt(ta, tb)}) OP ({op[0]}, {op[1]}, {op[2]})"
    return Configuration(name, conf, {"a": (K, M) if ta else (M, K), "b": (N, K) if tb else (K, N), "d": (M, N)},
                         {"a": cab, "b": cab, "d": ccd})


FPU_TYPES = [(T.Float16, T.Float16, T.Float32), (T.Float32, T.Float32, T.Float32), (T.Float32, T.Float32, T.Float64),
             (T.Float64, T.Float64, T.Float64), (T.Int16, T.Int16, T.Int16), (T.Int32, T.Int32, T.Int32),
             (T.Int64, T.Int64, T.Int64)]
FPU_OP_SHAPES = ([(m, n, k, 4, 8, 1) for m, n, k in [(4, 8, 1), (8, 8, 1), (4, 16, 1), (4, 8, 2), (8, 16, 2)]]
                 + [(4, 32, 1, 1, 32, 1), (4, 32, 1, 2, 16, 1), (16, 16, 1, 4, 8, 1), (16, 16, 1, 8, 4, 1),
                    (32, 4, 1, 16, 2, 1), (32, 4, 1, 32, 1, 1)])
WMMA_OPS = [(16, 16, 16), (8, 32, 16), (32, 8, 16)]
SQUARES = [(1, 1, 1), (2, 2, 1), (1, 1, 2), (2, 2, 2)]


def get_configs(largest: bool = True) -> list:
    """The list of configs.jl:492-690, ConfigError entries dropped as there.  `largest=False` leaves out
    the 2048 / 4096 cases (the quick list the CPU-side tests walk through)."""
    rv = []

    def push(make, *args, **kw):
        try:
            rv.append(make(*args, **kw))
        except ConfigError:
            pass

    tf = (False, True)
    for (A, B, CD), ta, tb, N in itertools.product(FPU_TYPES, tf, tf, [128, 256, 2048] if largest else [128, 256]):
        push(fpu_config, A, B, CD, ta, tb, (8, 16, 2, 4, 8, 1), (64, 64, 32), N, N, N)
    for ta, tb, op in itertools.product(tf, tf, FPU_OP_SHAPES):
        push(fpu_config, T.Float32, T.Float32, T.Float32, ta, tb, op, (128, 64, 32), 128, 128, 128)
    for ta, tb, (m, n, k) in itertools.product(tf, tf, SQUARES):
        push(fpu_config, T.Float32, T.Float32, T.Float32, ta, tb, (8, 16, 2, 4, 8, 1), (64, 64, 32),
             128 * m, 128 * n, 128 * k, tropical=True)
    for (AB, CD, md), ta, tb, op in itertools.product([(T.Float16, T.Float16, 256), (T.Float16, T.Float32, 128)], tf, tf, WMMA_OPS):
        sizes = [(md * m, md * n, md * k) for m, n, k in SQUARES] + ([(2048, 2048, 2048)] if largest else [])
        for M, N, K in sizes:
            push(wmma_config, AB, CD, ta, tb, (128, 128, 64), op, M, N, K)
    blocks = [b for b in itertools.product([64, 128, 256], [64, 128, 256], [16, 32, 64]) if b[0] * b[1] <= 128 * 128]
    # the parameter sweep of configs.jl:597-612: block shapes x warp grids x zero_c x kernels at 256^3
    warp_grids = [w for w in itertools.product([1, 2, 4], [1, 2, 4]) if w[0] * w[1] >= 4]
    for ta, tb, block, warps, zero_c, kern in itertools.product(tf, tf, blocks, warp_grids, tf,
                                                                [Kernel.matmul_singlestage, Kernel.matmul_pipelined]):
        push(wmma_config, T.Float16, T.Float32, ta, tb, block, (16, 16, 16), 256, 256, 256, zero_c=zero_c, kernel=kern, warps=warps)
    for ta, tb, op in itertools.product(tf, tf, WMMA_OPS):
        for M, N, K in [(128, 128, 128), (256, 256, 256)] + ([(4096, 4096, 4096)] if largest else []):
            push(wmma_bias_config, T.Float16, T.Float32, ta, tb, op, M, N, K)
    for tb, op in itertools.product(tf, WMMA_OPS):
        for M, N, K in [(128, 128, 128), (256, 256, 256)] + ([(4096, 4096, 4096)] if largest else []):
            push(wmma_diagonal_config, T.Float16, T.Float32, tb, op, M, N, K)
    cd_sizes = [(128, 128, 128), (256, 256, 256)] + ([(2048, 2048, 2048)] if largest else [])
    for ta, tb, op, (M, N, K) in itertools.product(tf, tf, WMMA_OPS, cd_sizes):
        push(wmma_complex_config, T.Float16, T.Float32, ta, tb, op, M, N, K)
    for op, (M, N, K) in itertools.product(WMMA_OPS, cd_sizes):
        push(wmma_complex_config, T.Float16, T.Float32, False, False, op, M, N, K, dual=True)
    # entries that differ only in a parameter the name does not show collapse, as they do in the
    # reference's results dictionary (keyed by name)
    seen, out = set(), []
    for c in rv:
        if c.name not in seen:
            seen.add(c.name)
            out.append(c)
    return out
