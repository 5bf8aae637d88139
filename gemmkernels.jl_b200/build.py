"""Builds libgemmkernels_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage:  python gemmkernels.jl_b200/build.py [--force] [--verbose]

The library has no dependency on libtorch or libcuda at link time (driver entry points are
resolved at run time through the CUDA runtime), so it can be loaded from Julia (`ccall`),
Python (`ctypes`) or C.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB_DIR = HERE / "lib"
LIB_PATH = LIB_DIR / "libgemmkernels_b200.so"

SOURCES = ["tc_kernels_rank3.cu", "tc_kernels_rank5.cu", "api.cu", "tc_plan.cu", "contract.cu", "mgpu.cu", "tc_kernels_generic.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.inc"))
    deps.append(HERE.parent / "include" / "gemmkernels_b200.h")
    deps.append(Path(__file__))
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library if any source is newer than it. Returns the path of the .so."""
    if not force and not _stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    def compile_one(src: str) -> str:
        obj = LIB_DIR / (Path(src).stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        return str(obj)

    # the translation units are independent: compile them side by side
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    cmd = [_nvcc(), "-shared", "-cudart", "static", "-o", str(LIB_PATH), *objs,
           "-Xlinker", "--exclude-libs=ALL", "-ldl"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
