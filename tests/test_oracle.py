"""CPU tests of the oracle itself: three independent restatements must agree with each other and
with the committed fixtures (tests/golden/golden_small.npz, made by tests/golden/make_golden.py).

The reference has no golden vectors for this path (its tests compare random inputs against an
independent product), so this is the strongest pin available: parity is "unpinned" against the
reference itself.
"""
import importlib.util
import math
from pathlib import Path

import numpy as np
import pytest

from oracle import c_oracle
from oracle import gemm_oracle as O

GOLDEN_DIR = Path(__file__).parent / "golden"


def _cases():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN_DIR / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.cases()


CASES = _cases()
GOLDEN = np.load(GOLDEN_DIR / "golden_small.npz")


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_golden(name):
    got, want = CASES[name]["D"], GOLDEN[f"{name}/D"]
    assert got.shape == want.shape and got.dtype == want.dtype
    if np.issubdtype(got.dtype, np.integer):
        assert np.array_equal(got, want)
    else:
        # BLAS builds may order sums differently: allow rounding noise of the accumulation type only
        assert O.normwise_error(got, want) <= (1e-12 if got.dtype == np.float64 else 2e-6)


def test_triple_loop_definition_agrees_with_blas_product():
    rng = np.random.default_rng(0)
    A = rng.standard_normal((7, 5)).astype(np.float32); B = rng.standard_normal((5, 9)).astype(np.float32)
    Cm = rng.standard_normal((7, 9)).astype(np.float32)
    loop = O.generic_mul(Cm, A, B, np.float32(2), np.float32(3))
    assert O.normwise_error(loop, O.gemm(A, B, Cm, 2.0, 3.0)) < 1e-6
    assert O.normwise_error(loop, c_oracle.gemm(A, B, Cm, 2.0, 3.0)) < 1e-6


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_c_restatement_agrees_with_numpy_fp32(ta, tb):
    rng = np.random.default_rng(1)
    M, N, K = 33, 29, 41
    A = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    B = rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    Cm = rng.standard_normal((M, N)).astype(np.float32)
    want = O.gemm64(A, B, Cm, 2.0, 3.0, ta, tb)
    assert O.normwise_error(c_oracle.gemm(A, B, Cm, 2.0, 3.0, ta, tb), want) < 1e-6
    assert O.normwise_error(c_oracle.gemm(A, B, Cm, 2.0, 3.0, ta, tb, f64_accumulate=True), want) < 1e-7
    assert O.normwise_error(O.gemm(A, B, Cm, 2.0, 3.0, ta, tb), want) < 1e-6


@pytest.mark.parametrize("dt", [np.int16, np.int32, np.int64])
def test_integer_gemm_wraps_like_the_c_loop(dt):
    rng = np.random.default_rng(2)
    info = np.iinfo(dt)
    A = rng.integers(info.min, info.max, (17, 13), dtype=dt); B = rng.integers(info.min, info.max, (13, 11), dtype=dt)
    Cm = rng.integers(info.min, info.max, (17, 11), dtype=dt)
    assert np.array_equal(O.integer_gemm(A, B, Cm, 2, 3), c_oracle.gemm(A, B, Cm, 2, 3))


def test_tropical_agrees_with_c_and_definition():
    case = CASES["tropical"]
    A, B, Cm = case["A"], case["B"], case["C"]
    assert np.array_equal(O.tropical_gemm(A, B, Cm), c_oracle.tropical(A, B, Cm))
    small = O.generic_mul(Cm[:5, :6].copy(), A[:5], B[:, :6], np.float32(1), np.float32(1),
                          element_update=lambda a, b, c: max(a + b, c))
    assert np.array_equal(small, O.tropical_gemm(A[:5], B[:, :6], Cm[:5, :6]))


def test_complex_and_dual_against_numpy_complex():
    A, B = CASES["complex_planar"]["A"].astype(np.float32), CASES["complex_planar"]["B"].astype(np.float32)
    z = (A[0] + 1j * A[1]).astype(np.complex128) @ (B[0] + 1j * B[1]).astype(np.complex128)
    re, im = O.complex_gemm(A[0], A[1], B[0], B[1])
    assert O.normwise_error(re, z.real) < 1e-6 and O.normwise_error(im, z.imag) < 1e-6
    # dual numbers: (a + a' eps)(b + b' eps) = ab + (ab' + a'b) eps
    re, du = O.dual_gemm(A[0], A[1], B[0], B[1])
    assert O.normwise_error(re, A[0].astype(np.float64) @ B[0]) < 1e-6
    assert O.normwise_error(du, A[0].astype(np.float64) @ B[1] + A[1].astype(np.float64) @ B[0]) < 1e-6


def test_contraction_is_a_permuted_gemm():
    A, B = CASES["contraction_aebf_dfce"]["A"], CASES["contraction_aebf_dfce"]["B"]
    e = A.shape[0]
    # M = (a, b), N = (c, d), K = (e, f)
    Am = A.astype(np.float32).transpose(0, 2, 1, 3).reshape(e * e, e * e)      # [a,b ; e,f]
    Bm = B.astype(np.float32).transpose(3, 1, 2, 0).reshape(e * e, e * e)      # [e,f ; c,d]
    want = (Am @ Bm).reshape(e, e, e, e)
    assert O.normwise_error(O.contract(A, "aebf", B, "dfce", "abcd"), want) < 1e-6


def test_bf16_and_tf32_rounding_helpers():
    x = np.array([1.0, 1.0 + 2 ** -8, 1.0 + 2 ** -7, 3.14159265, -2.71828], dtype=np.float32)
    r = O.bf16_round(x)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.0 + 2 ** -7)
    assert np.all(np.abs(r - x) <= np.abs(x) * 2 ** -8)
    t = O.tf32_truncate(x)
    assert np.all(np.abs(t - x) <= np.abs(x) * 2 ** -10) and np.all(np.abs(t) <= np.abs(x))


def test_comparison_rules_follow_the_reference():
    ref = np.array([1.0, 100.0, -3.0])
    assert O.isapprox_elementwise(ref, ref * (1 + 0.9 * math.sqrt(2.0 ** -10)), "Float16")
    assert not O.isapprox_elementwise(ref, ref * (1 + 1.5 * math.sqrt(2.0 ** -10)), "Float16")
    assert O.isapprox_elementwise(np.array([3, 4]), np.array([3, 4]), "Int32")
    assert not O.isapprox_elementwise(np.array([3, 4]), np.array([3, 5]), "Int32")
    assert O.isapprox_normwise(ref, ref + 1e-5, "Float32")
    assert O.normwise_error(ref * 1.001, ref) == pytest.approx(1e-3, rel=1e-6)
