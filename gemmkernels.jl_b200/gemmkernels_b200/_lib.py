"""ctypes binding of libgemmkernels_b200.so (declarations follow include/gemmkernels_b200.h).

There is no fallback: if the shared library is missing this module raises at import time, and
every compute call goes to the CUDA kernels.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("GEMMKERNELS_B200_LIB", _PKG.parent / "lib" / "libgemmkernels_b200.so"))

# --- enums (gemmkernels_b200.h) -------------------------------------------------------------
GK_OK, GK_ERR_INVALID_CONFIG, GK_ERR_UNSUPPORTED, GK_ERR_DIMENSION_MISMATCH = 0, 1, 2, 3
GK_ERR_CUDA, GK_ERR_TIMEOUT, GK_ERR_INVALID_ARGUMENT = 4, 5, 6

GK_F16, GK_BF16, GK_F32, GK_F64, GK_I16, GK_I32, GK_I64, GK_TF32 = range(8)
GK_OP_AUTO, GK_OP_TCGEN05, GK_OP_FPU, GK_OP_FPU_TROPICAL = range(4)
GK_REAL, GK_COMPLEX, GK_DUAL = range(3)
GK_LAYOUT_DENSE, GK_LAYOUT_ZERO, GK_LAYOUT_DIAGONAL = range(3)
GK_ACT_NONE, GK_ACT_RELU, GK_ACT_GELU = range(3)
GK_BIAS_NONE, GK_BIAS_ROW, GK_BIAS_COL = range(3)
GK_RASTER_AUTO, GK_RASTER_IDENTITY, GK_RASTER_HORIZONTAL, GK_RASTER_VERTICAL, GK_RASTER_LEBESGUE = range(5)

EXPORTS = (
    "gk_version", "gk_last_error_message", "gk_create", "gk_destroy", "gk_poll_status",
    "gk_gemm_query", "gk_gemm", "gk_gemm_host", "gk_contract_query", "gk_contract", "gk_debug_marks", "gk_measure_fp32_fma",
    "gk_contract_static",
    "gk_mgpu_unique_id", "gk_mgpu_init", "gk_mgpu_destroy", "gk_mgpu_gemm_colshard", "gk_mgpu_gemm_colshard_host",
    "gk_mgpu_host_plan", "gk_mgpu_broadcast", "gk_load_tuning",
)
GK_MGPU_UNIQUE_ID_BYTES = 128
GK_MGPU_A_RESIDENT, GK_MGPU_A_BROADCAST = 0, 1
GK_MAX_MODES = 8
GK_STATIC_TABLE_ENTRIES = 32768


class GemmDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("number", C.c_int32),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("trans_a", C.c_int32), ("trans_b", C.c_int32),
        ("dtype_a", C.c_int32), ("dtype_b", C.c_int32), ("dtype_c", C.c_int32), ("dtype_d", C.c_int32),
        ("compute", C.c_int32), ("op", C.c_int32),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("ldd", C.c_int64),
        ("plane_a", C.c_int64), ("plane_b", C.c_int64), ("plane_c", C.c_int64), ("plane_d", C.c_int64),
        ("layout_a", C.c_int32), ("layout_b", C.c_int32), ("layout_c", C.c_int32),
        ("raster", C.c_int32),
        ("alpha", C.c_double), ("beta", C.c_double),
        ("tile_n", C.c_int32), ("cta_group", C.c_int32), ("stages", C.c_int32),
        ("raster_group", C.c_int32), ("max_ctas", C.c_int32),
        ("debug", C.c_int32), ("host_chunk_mib", C.c_int32), ("a_resident", C.c_int32),
        ("batch", C.c_int32), ("k_blocks_per_stage", C.c_int32),
        ("batch_stride_a", C.c_int64), ("batch_stride_b", C.c_int64), ("batch_stride_c", C.c_int64),
        ("batch_stride_d", C.c_int64),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(GemmDesc)


class EpilogueDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("bias_axis", C.c_int32),
        ("bias", C.c_void_p),
        ("activation", C.c_int32), ("reserved", C.c_int32 * 3),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(EpilogueDesc)


class GemmPlan(C.Structure):
    _fields_ = [
        ("kernel", C.c_int32), ("grid", C.c_int32), ("block", C.c_int32), ("cluster", C.c_int32),
        ("smem_bytes", C.c_int32), ("tmem_columns", C.c_int32),
        ("tile_m", C.c_int32), ("tile_n", C.c_int32), ("tile_k", C.c_int32), ("stages", C.c_int32),
        ("workspace_bytes", C.c_int64),
    ]


class TuningEntry(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("trans_a", C.c_int32), ("trans_b", C.c_int32), ("has_c", C.c_int32),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("tile_n", C.c_int32), ("cta_group", C.c_int32), ("stages", C.c_int32), ("raster_group", C.c_int32),
        ("k_blocks_per_stage", C.c_int32), ("reserved", C.c_int32),
    ]


class MgpuTimes(C.Structure):
    _fields_ = [
        ("upload_ms", C.c_float), ("collective_ms", C.c_float), ("compute_ms", C.c_float), ("download_ms", C.c_float),
        ("total_ms", C.c_float), ("chunks", C.c_int32), ("reserved", C.c_int32),
        ("h2d_bytes", C.c_int64), ("d2h_bytes", C.c_int64),
    ]


class ContractDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("rank_a", C.c_int32), ("rank_b", C.c_int32), ("rank_c", C.c_int32),
        ("modes_a", C.c_int32 * 8), ("modes_b", C.c_int32 * 8), ("modes_c", C.c_int32 * 8),
        ("extents_a", C.c_int64 * 8), ("extents_b", C.c_int64 * 8), ("extents_c", C.c_int64 * 8),
        ("strides_a", C.c_int64 * 8), ("strides_b", C.c_int64 * 8), ("strides_c", C.c_int64 * 8),
        ("strides_d", C.c_int64 * 8),
        ("dtype_a", C.c_int32), ("dtype_b", C.c_int32), ("dtype_c", C.c_int32), ("dtype_d", C.c_int32),
        ("compute", C.c_int32), ("force_gather", C.c_int32),
        ("alpha", C.c_double), ("beta", C.c_double),
        ("tile_n", C.c_int32), ("cta_group", C.c_int32), ("stages", C.c_int32),
        ("debug", C.c_int32), ("reserved", C.c_int32 * 2),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(ContractDesc)


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python gemmkernels.jl_b200/build.py` "
            "(the package has no CPU or PyTorch fallback)")
    lib = C.CDLL(str(LIB_PATH))
    lib.gk_version.restype = C.c_int32
    lib.gk_version.argtypes = []
    lib.gk_last_error_message.restype = C.c_char_p
    lib.gk_last_error_message.argtypes = []
    lib.gk_create.restype = C.c_int
    lib.gk_create.argtypes = [C.POINTER(C.c_void_p)]
    lib.gk_destroy.restype = C.c_int
    lib.gk_destroy.argtypes = [C.c_void_p]
    lib.gk_poll_status.restype = C.c_int
    lib.gk_poll_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    lib.gk_gemm_query.restype = C.c_int
    lib.gk_gemm_query.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.POINTER(EpilogueDesc), C.POINTER(GemmPlan)]
    lib.gk_gemm.restype = C.c_int
    lib.gk_gemm.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                            C.c_void_p, C.POINTER(EpilogueDesc), C.c_void_p, C.c_int64, C.c_void_p]
    lib.gk_gemm_host.restype = C.c_int
    lib.gk_gemm_host.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.POINTER(EpilogueDesc), C.c_void_p]
    lib.gk_measure_fp32_fma.restype = C.c_int
    lib.gk_measure_fp32_fma.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.c_void_p]
    lib.gk_debug_marks.restype = C.c_int
    lib.gk_debug_marks.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    lib.gk_contract_query.restype = C.c_int
    lib.gk_contract_query.argtypes = [C.c_void_p, C.POINTER(ContractDesc), C.POINTER(GemmPlan)]
    lib.gk_contract.restype = C.c_int
    lib.gk_contract.argtypes = [C.c_void_p, C.POINTER(ContractDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    lib.gk_contract_static.restype = C.c_int
    lib.gk_contract_static.argtypes = [C.POINTER(ContractDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p]
    lib.gk_load_tuning.restype = C.c_int
    lib.gk_load_tuning.argtypes = [C.c_void_p, C.POINTER(TuningEntry), C.c_int32]
    lib.gk_mgpu_unique_id.restype = C.c_int
    lib.gk_mgpu_unique_id.argtypes = [C.c_void_p]
    lib.gk_mgpu_init.restype = C.c_int
    lib.gk_mgpu_init.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.gk_mgpu_destroy.restype = C.c_int
    lib.gk_mgpu_destroy.argtypes = [C.c_void_p]
    lib.gk_mgpu_gemm_colshard.restype = C.c_int
    lib.gk_mgpu_gemm_colshard.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(EpilogueDesc), C.c_void_p,
                                          C.c_int64, C.c_void_p]
    lib.gk_mgpu_gemm_colshard_host.restype = C.c_int
    lib.gk_mgpu_gemm_colshard_host.argtypes = [C.c_void_p, C.POINTER(GemmDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_void_p, C.POINTER(EpilogueDesc), C.c_void_p, C.POINTER(MgpuTimes)]
    lib.gk_mgpu_broadcast.restype = C.c_int
    lib.gk_mgpu_broadcast.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]
    lib.gk_mgpu_host_plan.restype = C.c_int
    lib.gk_mgpu_host_plan.argtypes = [C.POINTER(GemmDesc), C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int64)]
    return lib


lib = _load()


def last_error() -> str:
    return lib.gk_last_error_message().decode("utf-8", "replace")
