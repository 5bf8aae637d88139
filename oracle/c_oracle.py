"""ctypes binding of the C restatement (oracle/gemm_oracle.c) — TEST INFRASTRUCTURE ONLY.

Builds oracle/_build/liboracle.so with gcc on first use.  PARITY UNPINNED (see gemm_oracle.py).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "liboracle.so"


def build() -> Path:
    src = HERE / "gemm_oracle.c"
    if not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
    return _lib


_NAMES = {
    (np.dtype(np.float32), np.dtype(np.float32)): "oracle_gemm_f32",
    (np.dtype(np.float64), np.dtype(np.float64)): "oracle_gemm_f64",
    (np.dtype(np.int16), np.dtype(np.int16)): "oracle_gemm_i16",
    (np.dtype(np.int32), np.dtype(np.int32)): "oracle_gemm_i32",
    (np.dtype(np.int64), np.dtype(np.int64)): "oracle_gemm_i64",
}


def _f(x):
    return np.asfortranarray(x)


def gemm(A, B, C_=None, alpha=1.0, beta=0.0, trans_a=False, trans_b=False, f64_accumulate=False):
    """alpha*op(A)*op(B) + beta*C by the plain triple loop; A is stored (K, M) when trans_a."""
    A, B = _f(A), _f(B)
    M = A.shape[1] if trans_a else A.shape[0]
    K = A.shape[0] if trans_a else A.shape[1]
    N = B.shape[0] if trans_b else B.shape[1]
    out_dt = A.dtype if C_ is None else np.asarray(C_).dtype
    name = _NAMES[(A.dtype, np.dtype(out_dt))]
    if f64_accumulate and name == "oracle_gemm_f32":
        name = "oracle_gemm_f32_f64acc"
    D = np.zeros((M, N), dtype=out_dt, order="F")
    Cf = None if C_ is None else _f(np.asarray(C_))
    fn = getattr(lib(), name)
    fn.restype = None
    fn.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_double, C.c_void_p, C.c_int64,
                   C.c_void_p, C.c_int64, C.c_double, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64]
    fn(M, N, K, int(trans_a), int(trans_b), float(alpha), A.ctypes.data, A.shape[0], B.ctypes.data, B.shape[0],
       float(beta), None if Cf is None else Cf.ctypes.data, M, D.ctypes.data, M)
    return D


def tropical(A, B, C_=None, trans_a=False, trans_b=False):
    A, B = _f(np.asarray(A, dtype=np.float32)), _f(np.asarray(B, dtype=np.float32))
    M = A.shape[1] if trans_a else A.shape[0]
    K = A.shape[0] if trans_a else A.shape[1]
    N = B.shape[0] if trans_b else B.shape[1]
    D = np.zeros((M, N), dtype=np.float32, order="F")
    Cf = None if C_ is None else _f(np.asarray(C_, dtype=np.float32))
    fn = lib().oracle_tropical_f32
    fn.restype = None
    fn.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                   C.c_void_p, C.c_int64, C.c_void_p, C.c_int64]
    fn(M, N, K, int(trans_a), int(trans_b), A.ctypes.data, A.shape[0], B.ctypes.data, B.shape[0],
       None if Cf is None else Cf.ctypes.data, M, D.ctypes.data, M)
    return D
