"""pytest configuration: markers, import paths, shared helpers."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (ROOT, ROOT / "gemmkernels.jl_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


def _ensure_built():
    """The C-ABI library is built in-tree; build it if a source is newer (no GPU needed)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("gk_build", ROOT / "gemmkernels.jl_b200" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


_ensure_built()


@pytest.fixture(scope="session")
def gk():
    import gemmkernels_b200
    return gemmkernels_b200


@pytest.fixture(scope="session")
def oracle():
    from oracle import gemm_oracle
    return gemm_oracle
