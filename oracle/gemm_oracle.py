"""CPU oracle for the GEMM hot path — TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this file; the
product (gemmkernels.jl_b200/) never does and has no CPU path.

PARITY UNPINNED: the reference (GemmKernels.jl) holds no golden vectors or known-answer files for
this path — every check in its tests is "random inputs against an independent product"
(test/matmul.jl:12-20, test/blas.jl:21-36) — and it cannot be run here (no Julia, no CUDA.jl).
The oracle is therefore pinned only against itself: three independent restatements (the BLAS
product, a float64 product, and the plain C triple loop in gemm_oracle.c) must agree on the
committed fixtures under tests/golden/.

What each function restates (paths inside the GemmKernels.jl repository):
  generic_mul        configs/configs.jl:49-74   the alpha/beta triple loop that defines the math
  gemm / gemm64      LinearAlgebra.mul!(C, A, B, alpha, beta) on Float32-promoted inputs, the
                     comparator of test/blas.jl:34,63 and examples/simple_matmul.jl:55
  complex_gemm       src/operator.jl:301-314    re = ar*br - ai*bi, im = ar*bi + ai*br
  dual_gemm          src/operator.jl:360-372    re = ar*br, du = ar*bd + ad*br
  epilogue           src/epilogue.jl:44-73 and src/matmul.jl:196-200 (bias axis, order of ops)
  tropical_gemm      src/operator.jl:134-137    max-plus
  diagonal_gemm      src/layout.jl:225-236, configs/configs.jl:358-370   C += diag(v) * B
  contract           benchmarks/tensor-contractions/run.jl:137-155       einsum semantics
  isapprox_elementwise / normwise_error   configs/configs.jl:123-130, test/blas.jl:36,65
"""
from __future__ import annotations

import math

import numpy as np

# ------------------------------------------------------------------------------------------------
# element types
# ------------------------------------------------------------------------------------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    """Rounds float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def tf32_truncate(x: np.ndarray) -> np.ndarray:
    """FP32 values as the tensor cores read them in TF32 mode (10 explicit mantissa bits)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return (u & 0xFFFFE000).astype(np.uint32).view(np.float32)


# ------------------------------------------------------------------------------------------------
# the definition of the math: configs/configs.jl:49-74
# ------------------------------------------------------------------------------------------------
def generic_mul(C, A, B, alpha, beta, element_update=None):
    """res = beta*C[i,j]; for k: res = alpha * element_update(A[i,k], B[k,j], res).  With the
    default element_update (fma) and alpha folded once this is alpha*A*B + beta*C; the loop form
    is kept for the tropical variant, where alpha multiplies at every step.  Small sizes only."""
    M, N = C.shape
    K = A.shape[1]
    out = np.empty_like(C)
    for i in range(M):
        for j in range(N):
            if element_update is None:
                acc = C.dtype.type(0)
                for k in range(K):
                    acc = acc + A[i, k] * B[k, j]
                out[i, j] = alpha * acc + beta * C[i, j]
            else:
                res = beta * C[i, j]
                for k in range(K):
                    res = alpha * element_update(A[i, k], B[k, j], res)
                out[i, j] = res
    return out


def _op(X, trans):
    return X.T if trans else X


def gemm(A, B, C=None, alpha=1.0, beta=0.0, trans_a=False, trans_b=False, dtype=np.float32):
    """alpha * op(A) * op(B) + beta * C with inputs promoted to `dtype` (Float32 = the reference's
    CPU check; BLAS sgemm).  A is stored (K, M) when trans_a."""
    a = _op(np.asarray(A), trans_a).astype(dtype)
    b = _op(np.asarray(B), trans_b).astype(dtype)
    r = dtype(alpha) * (a @ b)
    if C is not None and beta != 0:
        r = r + dtype(beta) * np.asarray(C).astype(dtype)
    return r


def gemm64(A, B, C=None, alpha=1.0, beta=0.0, trans_a=False, trans_b=False):
    """Float64 product: the tight oracle for the FP32 (<= 1e-5) path."""
    return gemm(A, B, C, alpha, beta, trans_a, trans_b, dtype=np.float64)


def integer_gemm(A, B, C, alpha, beta, trans_a=False, trans_b=False):
    """Integer GEMM with wrap-around, as Julia's mul! on IntN arrays (compare exactly)."""
    dt = np.asarray(C).dtype
    a = _op(np.asarray(A), trans_a).astype(np.int64)
    b = _op(np.asarray(B), trans_b).astype(np.int64)
    with np.errstate(over="ignore"):
        r = np.int64(alpha) * (a @ b) + np.int64(beta) * np.asarray(C).astype(np.int64)
    return r.astype(dt)


def activation(x, name):
    if name in (None, "none"):
        return x
    if name == "relu":
        return np.maximum(x, 0)
    if name == "gelu":
        erf = np.vectorize(math.erf)
        return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))
    raise ValueError(name)


def epilogue(acc, bias=None, bias_axis="col", act=None):
    """D = act(acc + bias): the bias is added after the accumulator is scaled/combined with C and
    before the shared_to_global_d transform (src/epilogue.jl:67-70).  bias_axis 'col' = one value
    per column (the reference's layout, length N), 'row' = one per row (length M)."""
    x = acc
    if bias is not None:
        b = np.asarray(bias).reshape(-1).astype(acc.dtype)
        x = x + (b[None, :] if bias_axis == "col" else b[:, None])
    return activation(x, act)


def complex_gemm(Ar, Ai, Br, Bi, Cr=None, Ci=None, alpha=1.0, beta=0.0, trans_a=False, trans_b=False,
                 dtype=np.float32):
    """Planar complex product, four real GEMMs (src/operator.jl:301-314); transposes are plain
    transposes (no conjugation), as in configs/configs.jl:393-431."""
    g = lambda X, Y: gemm(X, Y, None, 1.0, 0.0, trans_a, trans_b, dtype)
    re = g(Ar, Br) - g(Ai, Bi)
    im = g(Ar, Bi) + g(Ai, Br)
    re, im = dtype(alpha) * re, dtype(alpha) * im
    if Cr is not None and beta != 0:
        re = re + dtype(beta) * np.asarray(Cr).astype(dtype)
        im = im + dtype(beta) * np.asarray(Ci).astype(dtype)
    return re, im


def dual_gemm(Ar, Ad, Br, Bd, Cr=None, Cd=None, alpha=1.0, beta=0.0, trans_a=False, trans_b=False,
              dtype=np.float32):
    """Dual-number product, three real GEMMs (src/operator.jl:360-372)."""
    g = lambda X, Y: gemm(X, Y, None, 1.0, 0.0, trans_a, trans_b, dtype)
    re = g(Ar, Br)
    du = g(Ar, Bd) + g(Ad, Br)
    re, du = dtype(alpha) * re, dtype(alpha) * du
    if Cr is not None and beta != 0:
        re = re + dtype(beta) * np.asarray(Cr).astype(dtype)
        du = du + dtype(beta) * np.asarray(Cd).astype(dtype)
    return re, du


def tropical_gemm(A, B, C=None, trans_a=False, trans_b=False):
    """Max-plus product with alpha = beta = 1 (configs/configs.jl:230-231):
    D[i,j] = max(C[i,j], max_k(A[i,k] + B[k,j]))."""
    a = _op(np.asarray(A), trans_a).astype(np.float32)
    b = _op(np.asarray(B), trans_b).astype(np.float32)
    M, K = a.shape
    out = np.full((M, b.shape[1]), -np.inf, dtype=np.float32) if C is None else np.asarray(C, dtype=np.float32).copy()
    for k in range(K):
        np.maximum(out, a[:, k:k + 1] + b[k:k + 1, :], out=out)
    return out


def diagonal_gemm(v, B, C):
    """C + diag(v) * B (src/layout.jl:225-236; the reference's harness ignores alpha and beta here,
    configs/configs.jl:363-370)."""
    return np.asarray(C, dtype=np.float32) + np.asarray(v, dtype=np.float32).reshape(-1, 1) * np.asarray(B, dtype=np.float32)


def contract(A, modes_a: str, B, modes_b: str, modes_c: str, alpha=1.0, beta=0.0, C=None, dtype=np.float32):
    """C[modes_c] = alpha * sum over shared modes of A[modes_a] * B[modes_b] (+ beta * C)."""
    r = dtype(alpha) * np.einsum(f"{modes_a},{modes_b}->{modes_c}", np.asarray(A).astype(dtype),
                                 np.asarray(B).astype(dtype), optimize=True)
    if C is not None and beta != 0:
        r = r + dtype(beta) * np.asarray(C).astype(dtype)
    return r


# ------------------------------------------------------------------------------------------------
# comparison rules
# ------------------------------------------------------------------------------------------------
def normwise_error(d, ref) -> float:
    """||d - ref||_F / ||ref||_F in float64."""
    d = np.asarray(d, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(d - ref) / den) if den > 0 else float(np.linalg.norm(d - ref))


_EPS = {"Float16": 2.0 ** -10, "BFloat16": 2.0 ** -7, "Float32": 2.0 ** -23, "Float64": 2.0 ** -52}


def isapprox_elementwise(ref, d, eltype_name: str) -> bool:
    """all(isapprox.(ref, d; rtol = sqrt(eps(T)))) with T = A's element type
    (configs/configs.jl:123-130); integers compare exactly."""
    if eltype_name.startswith("Int"):
        return bool(np.array_equal(ref, d))
    rtol = math.sqrt(_EPS[eltype_name])
    ref = np.asarray(ref, dtype=np.float64)
    d = np.asarray(d, dtype=np.float64)
    return bool(np.all(np.abs(ref - d) <= rtol * np.maximum(np.abs(ref), np.abs(d))))


def isapprox_normwise(ref, d, eltype_name: str) -> bool:
    """`ref ≈ d rtol = sqrt(eps(T))` on whole arrays (test/blas.jl:36,65)."""
    rtol = math.sqrt(_EPS[eltype_name])
    ref = np.asarray(ref, dtype=np.float64)
    d = np.asarray(d, dtype=np.float64)
    return bool(np.linalg.norm(ref - d) <= rtol * max(np.linalg.norm(ref), np.linalg.norm(d)))


# ------------------------------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations (values and distributions of each
# configuration; seeds 1000 + cfg for A, 2000 + cfg for B, 3000 + cfg for bias / C)
# ------------------------------------------------------------------------------------------------
def _rng(seed):
    return np.random.default_rng(seed)


def inputs_fp16_uniform01(cfg: int, M, N, K):
    """c0 / c1: A, B Float16 ~ U[0,1), column-major, C = 0."""
    A = _rng(1000 + cfg).random((M, K), dtype=np.float32).astype(np.float16)
    B = _rng(2000 + cfg).random((K, N), dtype=np.float32).astype(np.float16)
    return A, B


def inputs_fp32_bias_relu(cfg: int, M, N, K):
    """c2: A stored (K, M) (transposed), B (K, N), bias length M, all Float32 ~ N(0,1)."""
    At = _rng(1000 + cfg).standard_normal((K, M), dtype=np.float32)
    B = _rng(2000 + cfg).standard_normal((K, N), dtype=np.float32)
    bias = _rng(3000 + cfg).standard_normal((M,), dtype=np.float32)
    return At, B, bias


def inputs_planar_fp16(cfg: int, M, N, K):
    """c3: two Float16 planes per operand ~ U[-1,1)."""
    ra, rb = _rng(1000 + cfg), _rng(2000 + cfg)
    A = (ra.random((2, M, K), dtype=np.float32) * 2 - 1).astype(np.float16)
    B = (rb.random((2, K, N), dtype=np.float32) * 2 - 1).astype(np.float16)
    return A, B


def inputs_contraction(cfg: int, extent=32):
    """c4: A[a,e,b,f], B[d,f,c,e] Float16 ~ U[-1,1), all extents equal."""
    s = (extent,) * 4
    A = (_rng(1000 + cfg).random(s, dtype=np.float32) * 2 - 1).astype(np.float16)
    B = (_rng(2000 + cfg).random(s, dtype=np.float32) * 2 - 1).astype(np.float16)
    return A, B


def inputs_bf16_normal(cfg: int, M, N, K, std=0.02):
    """c5: A, B ~ N(0, 0.02) rounded to BFloat16 (returned as float32 holding bf16 values)."""
    A = bf16_round(_rng(1000 + cfg).standard_normal((M, K), dtype=np.float32) * np.float32(std))
    B = bf16_round(_rng(2000 + cfg).standard_normal((K, N), dtype=np.float32) * np.float32(std))
    return A, B
