"""gk_contract_static: the contraction entry point for callers that cannot allocate device memory
(their memory pool owns the whole GPU, or their callback contract forbids allocation).  It keeps the
gather kernel's offset tables in a fixed array inside the library instead of a caller workspace.

Checked here through the C ABI: its output equals the existing entry point's (gk_contract) on two
calls in a row that share the fixed array, and sizes beyond the array are refused with a clear
message.  This file sorts last on purpose, so a run that stops at the first failure has already
run every other test; it also passes on its own in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import gemmkernels_b200 as GK
from gemmkernels_b200 import _lib as L
from gemmkernels_b200.contract import _desc
from oracle import gemm_oracle as O

pytestmark = pytest.mark.gpu

TOL = 1e-3   # normwise, FP16 inputs with FP32 accumulation (same bound as the other contraction tests)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _run_both(A, modes_a, B, modes_b, modes_d, shape_d, alpha=1.0, beta=0.0, Cm=None):
    """Returns (static result, existing-entry result) as numpy arrays."""
    a, b = GK.to_cuarray(A), GK.to_cuarray(B)
    d_static = GK.to_cuarray(Cm) if Cm is not None else GK.cuarray(GK.Float32, *shape_d)
    d_ref = GK.to_cuarray(Cm) if Cm is not None else GK.cuarray(GK.Float32, *shape_d)
    desc = _desc(d_static, modes_d, a, modes_a, b, modes_b, alpha, beta, d_static if beta else None, None, False, 0, 0)
    st = L.lib.gk_contract_static(C.byref(desc), a.data_ptr(), b.data_ptr(),
                                  d_static.data_ptr() if beta else None, d_static.data_ptr(), _stream())
    assert st == L.GK_OK, L.last_error()
    # the existing entry point, on its default path (tensor cores when the modes allow, else gather)
    GK.contract_(d_ref, modes_d, a, modes_a, b, modes_b, alpha=alpha, beta=beta)
    torch.cuda.synchronize()
    GK.poll_status()
    return GK.to_numpy(d_static), GK.to_numpy(d_ref)


def test_static_contraction_matches_existing_entry_point_twice():
    rng = np.random.default_rng(41)
    # call 1: C[a,b,c,d] = sum_{e,f} A[a,e,b,f] B[d,f,c,e], extents 16 (M = N = K = 256)
    e = 16
    A = (rng.random((e, e, e, e)) * 2 - 1).astype(np.float16)
    B = (rng.random((e, e, e, e)) * 2 - 1).astype(np.float16)
    got, ref = _run_both(A, "aebf", B, "dfce", "abcd", (e, e, e, e))
    assert O.normwise_error(got, ref) <= TOL
    assert O.normwise_error(got, O.contract(A, "aebf", B, "dfce", "abcd")) <= TOL
    # call 2 right after it, a different and smaller contraction with alpha/beta: the fixed array still
    # holds call 1's longer tables, which must not leak into this result
    A2 = (rng.random((24, 40, 8)) * 2 - 1).astype(np.float16)       # A[b,d,a]
    B2 = (rng.random((40, 12)) * 2 - 1).astype(np.float16)          # B[d,c]
    C2 = rng.random((8, 24, 12)).astype(np.float32)                 # C[a,b,c]
    got2, ref2 = _run_both(A2, "bda", B2, "dc", "abc", (8, 24, 12), alpha=2.0, beta=0.5, Cm=C2)
    assert O.normwise_error(got2, ref2) <= TOL
    assert O.normwise_error(got2, O.contract(A2, "bda", B2, "dc", "abc", 2.0, 0.5, C2)) <= TOL
    # and call 1 again gives call 1's answer again
    got3, _ = _run_both(A, "aebf", B, "dfce", "abcd", (e, e, e, e))
    assert np.array_equal(got3, got)


def test_static_contraction_refuses_sizes_beyond_its_array():
    # M = N = K = 4608: 8 * 4608 = 36864 table entries > 32768
    n = 4608
    a = GK.cuarray(GK.Float16, n, n); b = GK.cuarray(GK.Float16, n, n); d = GK.cuarray(GK.Float32, n, n)
    desc = _desc(d, "ij", a, "ik", b, "kj", 1.0, 0.0, None, None, False, 0, 0)
    st = L.lib.gk_contract_static(C.byref(desc), a.data_ptr(), b.data_ptr(), None, d.data_ptr(), _stream())
    assert st == L.GK_ERR_INVALID_CONFIG
    msg = L.last_error()
    assert "36864" in msg and str(L.GK_STATIC_TABLE_ENTRIES) in msg and "gk_contract" in msg


def test_static_contraction_runs_when_the_tables_fill_the_array_exactly():
    """3*M + 3*N + 2*K == GK_STATIC_TABLE_ENTRIES: the largest case the fixed array holds is launched
    (a short K keeps it cheap) and must agree with gk_contract and with the oracle."""
    M = N = 5456
    K = 16
    assert 3 * M + 3 * N + 2 * K == L.GK_STATIC_TABLE_ENTRIES
    rng = np.random.default_rng(43)
    A = (rng.random((M, K)) * 2 - 1).astype(np.float16)
    B = (rng.random((K, N)) * 2 - 1).astype(np.float16)
    got, ref = _run_both(A, "ik", B, "kj", "ij", (M, N))
    assert O.normwise_error(got, ref) <= TOL
    assert O.normwise_error(got, O.gemm(A, B)) <= TOL
    # one entry more is refused
    a = GK.cuarray(GK.Float16, M + 1, K); b = GK.cuarray(GK.Float16, K, N); d = GK.cuarray(GK.Float32, M + 1, N)
    desc = _desc(d, "ij", a, "ik", b, "kj", 1.0, 0.0, None, None, False, 0, 0)
    assert L.lib.gk_contract_static(C.byref(desc), a.data_ptr(), b.data_ptr(), None, d.data_ptr(), _stream()) == L.GK_ERR_INVALID_CONFIG
