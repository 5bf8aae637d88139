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
    # gk_gemm_desc: 2*4 + 3*8 + 2*4 + 6*4 + 4*8 + 4*8 + 4*4 + 2*8 + 5*4 + 3*4 = 192
    assert ctypes.sizeof(_lib.GemmDesc) == 192
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
