"""The C-ABI library loads without a GPU and exports every function include/*.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = header.read_text()
        names += re.findall(r"GK_API\s+[\w\s\*]+?\b(gk_\w+)\s*\(", text)
    return names


def test_header_declares_entry_points():
    names = declared_functions()
    assert {"gk_create", "gk_destroy", "gk_gemm", "gk_gemm_query", "gk_last_error_message", "gk_version"} <= set(names)


@pytest.mark.parametrize("name", declared_functions())
def test_symbol_exported(name):
    from gemmkernels_b200 import _lib
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    assert getattr(lib, name) is not None


def test_binding_lists_every_declared_function():
    from gemmkernels_b200 import _lib
    assert set(_lib.EXPORTS) == set(declared_functions())


def test_version_and_error_string_without_gpu():
    from gemmkernels_b200 import _lib
    assert _lib.lib.gk_version() >= 1
    assert isinstance(_lib.last_error(), str)


def test_struct_sizes_match_header_layout():
    """The ctypes mirrors must have the C layout: the library rejects any other struct_size."""
    from gemmkernels_b200 import _lib
    # gk_gemm_desc: 2*4 + 3*8 + 2*4 + 6*4 + 4*8 + 4*8 + 4*4 + 2*8 + 8*4 + 2*4 + 4*8 = 232
    assert ctypes.sizeof(_lib.GemmDesc) == 232
    assert ctypes.sizeof(_lib.ContractDesc) == 4 * 4 + 3 * 8 * 4 + 7 * 8 * 8 + 6 * 4 + 2 * 8 + 6 * 4
    assert ctypes.sizeof(_lib.EpilogueDesc) == 32
    assert ctypes.sizeof(_lib.GemmPlan) == 48


def test_create_fails_loudly_without_gpu():
    """No CPU fallback: without a device gk_create reports a CUDA error instead of succeeding."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from gemmkernels_b200 import _lib
    h = ctypes.c_void_p()
    st = _lib.lib.gk_create(ctypes.byref(h))
    assert st == _lib.GK_ERR_CUDA and not h.value
    assert "failed" in _lib.last_error() or "sm_" in _lib.last_error()


def _desc(_lib, **kw):
    base = dict(number=0, m=64, n=64, k=64, dtype_a=_lib.GK_F16, dtype_b=_lib.GK_F16, dtype_c=_lib.GK_F32,
                dtype_d=_lib.GK_F32, compute=_lib.GK_F16, op=_lib.GK_OP_TCGEN05, lda=64, ldb=64, ldc=64, ldd=64, alpha=1.0)
    base.update(kw)
    return _lib.GemmDesc(**base)


@pytest.mark.parametrize("which,needle", [("a", "A is NULL"), ("b", "B is NULL"), ("d", "D is NULL"),
                                          ("c", "C is NULL"), ("bias", "bias pointer is NULL"),
                                          ("ws", "workspace_bytes")])
def test_null_pointers_come_back_as_status_codes(which, needle):
    """A missing operand must be refused on the host (GK_ERR_INVALID_ARGUMENT), never dereferenced
    on the device.  The checks run before anything touches a GPU, so they are testable here; the
    pointers below are never read."""
    from gemmkernels_b200 import _lib
    fake = ctypes.c_void_p(0x1000)
    ptr = {k: fake for k in "abcd"}
    desc = _desc(_lib, beta=1.0 if which == "c" else 0.0)
    epi = _lib.EpilogueDesc()
    ws, ws_bytes = None, 0
    if which in ptr:
        ptr[which] = None
    if which == "bias":
        epi.bias_axis = _lib.GK_BIAS_ROW
    if which == "ws":
        ws_bytes = 1024
    for call in ("gk_gemm", "gk_gemm_host"):
        if call == "gk_gemm":
            st = _lib.lib.gk_gemm(None, ctypes.byref(desc), ptr["a"], ptr["b"], ptr["c"], ptr["d"], ctypes.byref(epi),
                                  ws, ws_bytes, None)
        else:
            if which == "ws":
                continue
            st = _lib.lib.gk_gemm_host(None, ctypes.byref(desc), ptr["a"], ptr["b"], ptr["c"], ptr["d"],
                                       ctypes.byref(epi), None)
        assert st == _lib.GK_ERR_INVALID_ARGUMENT, (call, _lib.last_error())
        assert needle in _lib.last_error(), (call, _lib.last_error())


def test_contract_with_beta_needs_c():
    from gemmkernels_b200 import _lib
    desc = _lib.ContractDesc(rank_a=2, rank_b=2, rank_c=2, alpha=1.0, beta=0.5)
    fake = ctypes.c_void_p(0x1000)
    st = _lib.lib.gk_contract(None, ctypes.byref(desc), fake, fake, None, fake, None, 0, None)
    assert st == _lib.GK_ERR_INVALID_ARGUMENT and "C is NULL" in _lib.last_error()
    st = _lib.lib.gk_contract_static(ctypes.byref(desc), fake, fake, None, fake, None)
    assert st == _lib.GK_ERR_INVALID_ARGUMENT and "C is NULL" in _lib.last_error()


def test_batched_descriptor_rules():
    from gemmkernels_b200 import _lib
    fake = ctypes.c_void_p(0x1000)
    desc = _desc(_lib, batch=4, batch_stride_a=64 * 64, batch_stride_b=64 * 64, batch_stride_d=64 * 32)
    st = _lib.lib.gk_gemm(None, ctypes.byref(desc), fake, fake, None, fake, None, None, 0, None)
    assert st == _lib.GK_ERR_DIMENSION_MISMATCH and "overlap" in _lib.last_error()
    desc = _desc(_lib, batch=4, number=_lib.GK_COMPLEX, batch_stride_d=64 * 64)
    st = _lib.lib.gk_gemm(None, ctypes.byref(desc), fake, fake, None, fake, None, None, 0, None)
    assert st == _lib.GK_ERR_INVALID_CONFIG
