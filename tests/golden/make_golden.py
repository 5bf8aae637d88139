"""Generates tests/golden/golden_small.npz from the CPU oracle (run from the repository root:
`python tests/golden/make_golden.py`).

The reference holds no golden vectors and cannot run in this environment, so these fixtures pin
the oracle against itself over time (numpy/BLAS, float64 and the C triple loop must keep agreeing
with what is stored here); they are small seeded cases shaped like the benchmark configurations.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import gemm_oracle as O  # noqa: E402


def cases():
    """name -> (inputs dict, expected dict).  Inputs are regenerated from seeds by the tests; only
    their shapes/seeds matter here, but they are stored too so the file is self-contained."""
    out = {}
    # mixed-precision GEMM, U[0,1) FP16 (shape of configuration 1, scaled down)
    A, B = O.inputs_fp16_uniform01(1, 96, 80, 72)
    out["fp16_nn"] = dict(A=A, B=B, D=O.gemm(A, B))
    # alpha/beta and both operands transposed
    rng = np.random.default_rng(7)
    At = rng.random((72, 96), dtype=np.float32).astype(np.float16)
    Bt = rng.random((80, 72), dtype=np.float32).astype(np.float16)
    C = rng.random((96, 80), dtype=np.float32)
    out["fp16_tt_alpha_beta"] = dict(A=At, B=Bt, C=C, D=O.gemm(At, Bt, C, 2.0, 3.0, True, True))
    # FP32, A transposed, row bias + ReLU (configuration 2, scaled down)
    At, B, bias = O.inputs_fp32_bias_relu(2, 88, 104, 64)
    out["fp32_tn_bias_relu"] = dict(A=At, B=B, bias=bias,
                                    D=O.epilogue(O.gemm64(At, B, trans_a=True), bias, "row", "relu"))
    out["fp32_tn_colbias_gelu"] = dict(A=At, B=B, bias=np.arange(104, dtype=np.float32) / 50 - 1,
                                       D=O.epilogue(O.gemm64(At, B, trans_a=True),
                                                    np.arange(104, dtype=np.float32) / 50 - 1, "col", "gelu"))
    # planar complex and dual (configuration 3, scaled down)
    A, B = O.inputs_planar_fp16(3, 128, 64, 96)
    re, im = O.complex_gemm(A[0], A[1], B[0], B[1])
    out["complex_planar"] = dict(A=A, B=B, D=np.stack([re, im]))
    re, du = O.dual_gemm(A[0], A[1], B[0], B[1])
    out["dual_planar"] = dict(A=A, B=B, D=np.stack([re, du]))
    # tensor contraction C[a,b,c,d] = sum_{e,f} A[a,e,b,f] B[d,f,c,e] (configuration 4, extents 8)
    A, B = O.inputs_contraction(4, 8)
    out["contraction_aebf_dfce"] = dict(A=A, B=B, D=O.contract(A, "aebf", B, "dfce", "abcd"))
    # BF16 N(0, 0.02) (configuration 5, scaled down)
    A, B = O.inputs_bf16_normal(5, 80, 96, 112)
    out["bf16_nn"] = dict(A=A, B=B, D=O.gemm(A, B))
    # integers wrap around
    rng = np.random.default_rng(11)
    A = rng.integers(-2 ** 31, 2 ** 31 - 1, (40, 56), dtype=np.int32)
    B = rng.integers(-2 ** 31, 2 ** 31 - 1, (56, 24), dtype=np.int32)
    C = rng.integers(-2 ** 31, 2 ** 31 - 1, (40, 24), dtype=np.int32)
    out["int32_wrap"] = dict(A=A, B=B, C=C, D=O.integer_gemm(A, B, C, 2, 3))
    # max-plus
    rng = np.random.default_rng(13)
    A = rng.random((48, 40), dtype=np.float32); B = rng.random((40, 56), dtype=np.float32)
    C = rng.random((48, 56), dtype=np.float32) + 0.5
    out["tropical"] = dict(A=A, B=B, C=C, D=O.tropical_gemm(A, B, C))
    # diagonal A
    rng = np.random.default_rng(17)
    v = rng.random(64, dtype=np.float32).astype(np.float16); B = rng.random((64, 40), dtype=np.float32).astype(np.float16)
    C = rng.random((64, 40), dtype=np.float32)
    out["diagonal"] = dict(A=v, B=B, C=C, D=O.diagonal_gemm(v, B, C))
    return out


if __name__ == "__main__":
    # Only the expected outputs are stored; tests regenerate the inputs from the same seeds.
    flat = {f"{name}/D": arrs["D"] for name, arrs in cases().items()}
    path = Path(__file__).with_name("golden_small.npz")
    np.savez_compressed(path, **flat)
    print(path, path.stat().st_size, "bytes,", len(flat), "arrays")
