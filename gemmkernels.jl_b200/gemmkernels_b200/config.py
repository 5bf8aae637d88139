"""get_config / Config / ConfigError — host mirror of src/config.jl.

The 24 reference parameters are kept (tests and the tuner read them); the B200 engine adds
`tile_n`, `cta_group`, `stages`, `raster_group`.  Legacy parameters that described how warps of
the WMMA kernels split a tile (warps_per_block, mem_*_warp, compute_warp, ...) are validated by
the reference's own rules and then act as hints only.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from . import cta_swizzle as CTASwizzle
from . import layout as Layout
from . import operator as Operator


class ConfigError(Exception):
    """GemmKernels.ConfigError (src/config.jl:78-82)."""

    def __str__(self):
        return "ConfigError: " + super().__str__()


class DimensionMismatch(Exception):
    """Julia's DimensionMismatch (thrown by create_config, src/matmul.jl:75-77)."""


def _mnk(x, names="MNK"):
    if isinstance(x, dict):
        return {k: int(v) for k, v in x.items()}
    return {n: int(v) for n, v in zip(names, x)}


@dataclass
class Config:
    # src/config.jl:3-41 -----------------------------------------------------------------------
    matmul_shape: dict
    block_shape: dict
    warps_per_block: int
    mem_a_warp: dict
    mem_a_thread: dict
    mem_b_warp: dict
    mem_b_thread: dict
    mem_cd_warp: dict
    mem_cd_thread: dict
    compute_warp: dict
    compute_op_shape: dict
    global_a_layout: Any
    global_b_layout: Any
    global_c_layout: Any
    global_d_layout: Any
    shared_a_layout: Any
    shared_b_layout: Any
    shared_c_layout: Any
    shared_d_layout: Any
    operator: Any
    is_a_col_major: bool
    is_b_col_major: bool
    cta_swizzle: Any
    # B200 engine parameters (0 = take the built-in table) --------------------------------------
    tile_n: int = 0
    cta_group: int = 0
    stages: int = 0
    raster_group: int = 0
    k_blocks_per_stage: int = 0
    extra: dict = field(default_factory=dict)

    def __str__(self):
        rows = [(k, getattr(self, k)) for k in self.__dataclass_fields__ if k != "extra"]
        return "\n".join(f"{k + ':':<18}{v}" for k, v in rows)


def heuristic_block_shape(shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout):
    """src/config.jl:84-120: grow M, N alternately while a C/D tile fits 64 KiB, then K while
    A + B tiles fit 64 KiB."""
    def nbytes(layout, shape):
        n = 1
        for s in layout.physical_size(shape):
            n *= s
        return n * layout.eltype.size * (2 if getattr(layout.eltype, "is_complex", False) else 1)

    def fits_cd(m, n, k):
        return max(nbytes(shared_c_layout, (m, n)), nbytes(shared_d_layout, (m, n))) <= 64 * 1024

    def fits_ab(m, n, k):
        return nbytes(shared_a_layout, (m, k)) + nbytes(shared_b_layout, (k, n)) <= 64 * 1024

    def next_mn(m, n, k):
        return (2 * m, n, k) if m == n else (m, 2 * n, k)

    cur = (1, 1, 1)
    nxt = next_mn(*cur)
    while fits_cd(*nxt):
        cur, nxt = nxt, next_mn(*nxt)
    nxt = (cur[0], cur[1], 2 * cur[2])
    while fits_ab(*nxt):
        cur, nxt = nxt, (nxt[0], nxt[1], 2 * nxt[2])
    return {"M": cur[0], "N": cur[1], "K": cur[2]}


def adjacent_elements(num, parent_size: dict, is_col_major: bool) -> dict:
    """src/config.jl:124-134."""
    keys = list(parent_size.keys())
    p = [parent_size[k] for k in keys]
    if is_col_major:
        t = (min(num, p[0]), num // min(num, p[0]))
    else:
        t = (num // min(num, p[1]), min(num, p[1]))
    return {keys[0]: t[0], keys[1]: t[1]}


def check_operator_config(op) -> None:
    """src/config.jl:136-173."""
    if isinstance(op, Operator.FPUOp):
        s = op.base_shape()
        if s["M"] * s["N"] < 32:
            raise ConfigError("The operator shape is too small. The dimensions of the operator shape must adhere "
                              "to the following constraint: OPERATOR_M * OPERATOR_N ≥ 32.")
        if s["mb"] * s["nb"] != 32:
            raise ConfigError("The base FPU operator shape should adhere to the following constraint: "
                              "OPERATOR_M_BASE * OPERATOR_N_BASE = 32.")
        if s["kb"] != 1:
            raise ConfigError("The base FPU operator shape should adhere to the following constraint: OPERATOR_K_BASE = 1.")
        if s["M"] % s["mb"] or s["N"] % s["nb"] or s["K"] % s["kb"]:
            raise ConfigError("The operator shape should adhere to the following constraint: OPERATOR_M, OPERATOR_N, "
                              "OPERATOR_K are multiples of OPERATOR_M_BASE, OPERATOR_N_BASE, OPERATOR_K_BASE, respectively.")
    elif isinstance(op, Operator.WMMAOp):
        if (op.M, op.N, op.K) not in ((16, 16, 16), (8, 32, 16), (32, 8, 16)):
            raise ConfigError(f"Unsupported WMMA Operator shape (M = {op.M}, N = {op.N}, K = {op.K})!")
    elif isinstance(op, Operator.TCGen05Operator):
        ct = getattr(op.CT, "name", str(op.CT))
        if ct not in ("Float16", "BFloat16", "TF32"):
            raise ConfigError(f"TCGen05Operator computes in Float16, BFloat16 or TF32, not {ct}")
        if getattr(op.AT, "name", "") not in ("Float32", "Float16", "BFloat16"):
            raise ConfigError(f"TCGen05Operator accumulates in Float32 (stored as Float32/Float16/BFloat16), not {op.AT}")


def require_tile_sized_global(layout) -> bool:
    """src/config.jl:175-178."""
    base = layout.base
    return not isinstance(base, (Layout.Zero, Layout.ColMajor, Layout.RowMajor))


def get_config(*, gemm_shape, operator, global_a_layout, global_c_layout, **params) -> Config:
    """GemmKernels.get_config (src/config.jl:180-316): same keywords, same defaults, same errors."""
    gemm_shape = _mnk(gemm_shape)
    global_b_layout = params.get("global_b_layout", global_a_layout)
    global_d_layout = params.get("global_d_layout", global_c_layout)

    def esize(layout):
        return layout.eltype.size * (2 if getattr(layout.eltype, "is_complex", False) else 1)

    shared_a_layout = params.get("shared_a_layout", Layout.Padded(global_a_layout, 16 // esize(global_a_layout)))
    shared_b_layout = params.get("shared_b_layout", Layout.Padded(global_b_layout, 16 // esize(global_b_layout)))
    shared_c_layout = params.get("shared_c_layout", global_c_layout)
    shared_d_layout = params.get("shared_d_layout", global_d_layout)

    block_shape = params.get("block_shape")
    block_shape = _mnk(block_shape) if block_shape is not None else heuristic_block_shape(
        shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout)

    if block_shape["M"] * block_shape["K"] < 128 or block_shape["K"] * block_shape["N"] < 128 or block_shape["K"] < 8:
        raise ConfigError("The block shape is too small. The dimensions of the block shape must adhere to the following "
                          "constraints: BLOCK_M * BLOCK_K ≥ 128, BLOCK_K * BLOCK_N ≥ 128, BLOCK_K ≥ 8.")
    op_shape = operator.shape()
    if block_shape["M"] < 2 * op_shape["M"] or block_shape["N"] < 2 * op_shape["N"] or block_shape["K"] < op_shape["K"]:
        raise ConfigError("There is a mismatch between the block shape and the operator shape. Their dimensions must adhere "
                          "to the following constraints: BLOCK_M ≥ 2 * OPERATOR_M, BLOCK_N ≥ 2 * OPERATOR_N, BLOCK_K ≥ OPERATOR_K.")
    check_operator_config(operator)

    warps_default = 8
    compute_warp_default = {"M": block_shape["M"] // 4, "N": block_shape["N"] // 2, "K": op_shape["K"]}
    if block_shape["M"] // op_shape["M"] < 4 or block_shape["N"] // op_shape["N"] < 2:
        compute_warp_default = {"M": max(op_shape["M"], block_shape["M"] // 4),
                                "N": max(op_shape["N"], block_shape["N"] // 2), "K": op_shape["K"]}
        warps_default = min(block_shape["M"] // op_shape["M"], 4) * min(block_shape["N"] // op_shape["N"], 2)
    warps_per_block = int(params.get("warps_per_block", warps_default))
    compute_warp = _mnk(params.get("compute_warp", compute_warp_default))

    is_a_col_major = bool(params.get("is_a_col_major", True))
    is_b_col_major = bool(params.get("is_b_col_major", True))
    is_cd_col_major = bool(params.get("is_cd_col_major", True))

    bm, bn, bk = block_shape["M"], block_shape["N"], block_shape["K"]
    n_a = min(16 // esize(global_a_layout), (bm * bk) // (32 * warps_per_block))
    n_b = min(16 // esize(global_b_layout), (bk * bn) // (32 * warps_per_block))
    n_c = min(16 // esize(global_c_layout), (bm * bn) // (32 * warps_per_block))
    if min(n_a, n_b, n_c) < 1:
        raise ConfigError("mem_a_warp is too big for the selected block shape: need at least one iteration in the memory copy loop!")

    def named(x, names):
        return _mnk(x, names) if x is not None else None

    mem_a_warp = named(params.get("mem_a_warp"), "MK") or adjacent_elements(32 * n_a, {"M": bm, "K": bk}, is_a_col_major)
    mem_b_warp = named(params.get("mem_b_warp"), "KN") or adjacent_elements(32 * n_b, {"K": bk, "N": bn}, is_b_col_major)
    mem_cd_warp = named(params.get("mem_cd_warp"), "MN") or adjacent_elements(32 * n_c, {"M": bm, "N": bn}, is_cd_col_major)
    mem_a_thread = named(params.get("mem_a_thread"), "MK") or adjacent_elements(n_a, {"M": bm, "K": bk}, is_a_col_major)
    mem_b_thread = named(params.get("mem_b_thread"), "KN") or adjacent_elements(n_b, {"K": bk, "N": bn}, is_b_col_major)
    mem_cd_thread = named(params.get("mem_cd_thread"), "MN") or adjacent_elements(n_c, {"M": bm, "N": bn}, is_cd_col_major)

    def prod(d):
        r = 1
        for v in d.values():
            r *= v
        return r

    if prod(mem_a_warp) * warps_per_block > bm * bk:
        raise ConfigError("mem_a_warp is too big for the selected block shape: need at least one iteration in the memory copy loop!")
    if prod(mem_b_warp) * warps_per_block > bk * bn:
        raise ConfigError("mem_b_warp is too big for the selected block shape: need at least one iteration in the memory copy loop!")
    if prod(mem_cd_warp) * warps_per_block > bm * bn:
        raise ConfigError("mem_cd_warp is too big for the selected block shape: need at least one iteration in the memory copy loop!")

    def check_multiple(num, den, dims, msg):
        if any(num[d] % den[d] for d in dims):
            raise ConfigError(msg)

    check_multiple(block_shape, compute_warp, "MNK", "block_shape must be a multiple of compute_warp!")
    check_multiple(compute_warp, op_shape, "MNK", "compute_warp must be a multiple of op_shape!")
    if require_tile_sized_global(global_a_layout):
        check_multiple(gemm_shape, block_shape, "MK", "gemm_shape.MK must be a multiple of block_shape.MK!")
    if require_tile_sized_global(global_b_layout):
        check_multiple(gemm_shape, block_shape, "KN", "gemm_shape.KN must be a multiple of block_shape.KN!")
    if require_tile_sized_global(global_c_layout):
        check_multiple(gemm_shape, block_shape, "MN", "gemm_shape.MN must be a multiple of block_shape.MN!")
    if require_tile_sized_global(global_d_layout):
        check_multiple(gemm_shape, block_shape, "MN", "gemm_shape.MN must be a multiple of block_shape.MN!")

    tile_n = int(params.get("tile_n", 0))
    cta_group = int(params.get("cta_group", 0))
    if cta_group not in (0, 1, 2):
        raise ConfigError("cta_group must be 1 or 2 (0 = choose)")
    if tile_n and tile_n != 512 and (tile_n % 32 or not 32 <= tile_n <= 256):
        raise ConfigError("tile_n must be a multiple of 32 between 32 and 256, or 512 (0 = choose)")

    return Config(
        gemm_shape, block_shape, warps_per_block,
        mem_a_warp, mem_a_thread, mem_b_warp, mem_b_thread, mem_cd_warp, mem_cd_thread,
        compute_warp, op_shape,
        global_a_layout, global_b_layout, global_c_layout, global_d_layout,
        shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout,
        operator, is_a_col_major, is_b_col_major,
        params.get("cta_swizzle", CTASwizzle.Identity()),
        tile_n=tile_n, cta_group=cta_group, stages=int(params.get("stages", 0)),
        raster_group=int(params.get("raster_group", 0)),
        k_blocks_per_stage=int(params.get("k_blocks_per_stage", 0)),
    )
