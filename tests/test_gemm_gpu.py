"""GPU parity tests: the CUDA path, called through the C ABI (ctypes) by the host mirror of the
GemmKernels.jl API, against the CPU oracle on the same seeded inputs.

Tolerances: normwise relative error <= 1e-3 for the FP16/BF16/TF32 -> FP32 tensor-core paths and
<= 1e-5 for the FP32 FPU path (against a float64 product), plus the reference's own rules where its
test matrix is replayed: elementwise rtol = sqrt(eps(T)) (configs/configs.jl:123-130) and normwise
sqrt(eps(T)) (test/blas.jl:36,65).  Integer results must be bit-exact.
"""
import ctypes as C
import importlib.util
import itertools
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import gemmkernels_b200 as GK
from gemmkernels_b200 import CTASwizzle, _lib as L
from gemmkernels_b200 import Epilogue, Kernel, Layout, Operator, Transform
from oracle import gemm_oracle as O

pytestmark = pytest.mark.gpu

TOL_TENSOR = 1e-3
TOL_FPU = 1e-5
GOLDEN_DIR = Path(__file__).parent / "golden"


def _golden_cases():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN_DIR / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.cases()


@pytest.fixture(scope="module")
def golden():
    return _golden_cases(), np.load(GOLDEN_DIR / "golden_small.npz")


def dev(x, eltype=None):
    return GK.to_cuarray(np.asarray(x), eltype)


def planar(x, eltype=None):
    """numpy (2, r, c) planes -> device (r, c, 2) column-major planes (Layout.Split*)."""
    t = torch.from_numpy(np.ascontiguousarray(np.asarray(x).transpose(0, 2, 1)))   # [2, c, r]
    if eltype is not None:
        t = t.to(eltype.torch_dtype())
    return t.cuda().permute(2, 1, 0)


def run_matmul(a, b, c, d, *, M, N, K, op, la, lb, lc, ld, alpha=1.0, beta=1.0, epilogue=None, act=None,
               kernel=Kernel.matmul_singlestage, **conf_kw):
    conf = GK.get_config(gemm_shape=(M, N, K), operator=op, global_a_layout=la, global_b_layout=lb,
                         global_c_layout=lc, global_d_layout=ld, is_a_col_major=la.col_major,
                         is_b_col_major=lb.col_major, **conf_kw)
    kw = {}
    if alpha != 1.0:
        kw["transform_shared_to_regs_a"] = Transform.Elementwise(Transform.Scale(alpha))
    if beta != 1.0:
        kw["transform_shared_to_regs_c"] = Transform.Elementwise(Transform.Scale(beta))
    if act is not None:
        kw["transform_shared_to_global_d"] = Transform.Elementwise(act)
    GK.matmul(conf, a, b, c, d, epilogue=epilogue, kernel=kernel, **kw)
    torch.cuda.synchronize()
    GK.poll_status()
    return conf


# ------------------------------------------------------------------------------------------------
# committed golden fixtures
# ------------------------------------------------------------------------------------------------
def test_golden_fp16_nn(golden):
    cases, want = golden
    A, B = cases["fp16_nn"]["A"], cases["fp16_nn"]["B"]
    M, K = A.shape; N = B.shape[1]
    d = GK.cuarray(GK.Float32, M, N)
    run_matmul(dev(A), dev(B), None, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[GK.Float16, GK.Float32],
               la=Layout.ColMajor[GK.Float16], lb=Layout.ColMajor[GK.Float16],
               lc=Layout.Zero[GK.Float32], ld=Layout.ColMajor[GK.Float32], block_shape=(128, 128, 64))
    assert O.normwise_error(GK.to_numpy(d), want["fp16_nn/D"]) <= TOL_TENSOR


def test_golden_fp16_tt_alpha_beta(golden):
    cases, want = golden
    cs = cases["fp16_tt_alpha_beta"]
    At, Bt, Cm = cs["A"], cs["B"], cs["C"]
    K, M = At.shape; N = Bt.shape[0]
    c = dev(Cm); d = GK.cuarray(GK.Float32, M, N)
    run_matmul(dev(At), dev(Bt), c, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[GK.Float16, GK.Float32],
               la=Layout.RowMajor[GK.Float16], lb=Layout.RowMajor[GK.Float16],
               lc=Layout.ColMajor[GK.Float32], ld=Layout.ColMajor[GK.Float32], alpha=2.0, beta=3.0,
               block_shape=(128, 128, 64))
    assert O.normwise_error(GK.to_numpy(d), want["fp16_tt_alpha_beta/D"]) <= TOL_TENSOR


@pytest.mark.parametrize("case,axis,act", [("fp32_tn_bias_relu", "row", Transform.ReLU()),
                                           ("fp32_tn_colbias_gelu", "col", Transform.GELU())])
def test_golden_fp32_fpu_bias_activation(golden, case, axis, act):
    cases, want = golden
    cs = cases[case]
    At, B, bias = cs["A"], cs["B"], cs["bias"]
    K, M = At.shape; N = B.shape[1]
    d = GK.cuarray(GK.Float32, M, N)
    run_matmul(dev(At), dev(B), None, d, M=M, N=N, K=K, op=Operator.FPUOp[8, 8, 1, 4, 8, 1, GK.Float32, GK.Float32],
               la=Layout.RowMajor[GK.Float32], lb=Layout.ColMajor[GK.Float32],
               lc=Layout.Zero[GK.Float32], ld=Layout.ColMajor[GK.Float32],
               epilogue=Epilogue.Bias(dev(bias), axis=axis), act=act, block_shape=(128, 128, 32))
    assert O.normwise_error(GK.to_numpy(d), want[f"{case}/D"]) <= TOL_FPU


@pytest.mark.parametrize("case,opcls", [("complex_planar", Operator.WMMAComplexOp), ("dual_planar", Operator.WMMADualOp)])
def test_golden_planar_complex_and_dual(golden, case, opcls):
    cases, want = golden
    A, B = cases[case]["A"], cases[case]["B"]          # (2, M, K), (2, K, N)
    M, K = A.shape[1:]; N = B.shape[2]
    d = GK.cuarray(GK.Float32, M, N, 2)
    run_matmul(planar(A), planar(B), None, d, M=M, N=N, K=K, op=opcls[16, 16, 16, GK.Float16, GK.Float32],
               la=Layout.SplitColMajor[GK.Float16], lb=Layout.SplitColMajor[GK.Float16],
               lc=Layout.Zero[GK.Float32], ld=Layout.SplitColMajor[GK.Float32], block_shape=(64, 64, 32))
    got = GK.to_numpy(d).transpose(2, 0, 1)
    assert O.normwise_error(got, want[f"{case}/D"]) <= TOL_TENSOR


def test_golden_bf16(golden):
    cases, want = golden
    A, B = cases["bf16_nn"]["A"], cases["bf16_nn"]["B"]
    M, K = A.shape; N = B.shape[1]
    d = GK.cuarray(GK.Float32, M, N)
    run_matmul(dev(A, GK.BFloat16), dev(B, GK.BFloat16), None, d, M=M, N=N, K=K,
               op=Operator.TCGen05Operator[GK.BFloat16, GK.Float32],
               la=Layout.ColMajor[GK.BFloat16], lb=Layout.ColMajor[GK.BFloat16],
               lc=Layout.Zero[GK.Float32], ld=Layout.ColMajor[GK.Float32], block_shape=(128, 128, 64))
    assert O.normwise_error(GK.to_numpy(d), want["bf16_nn/D"]) <= TOL_TENSOR


def test_golden_int32_is_bit_exact(golden):
    cases, want = golden
    cs = cases["int32_wrap"]
    A, B, Cm = cs["A"], cs["B"], cs["C"]
    M, K = A.shape; N = B.shape[1]
    c = dev(Cm); d = GK.cuarray(GK.Int32, M, N)
    run_matmul(dev(A), dev(B), c, d, M=M, N=N, K=K, op=Operator.FPUOp[8, 16, 2, 4, 8, 1, GK.Int32, GK.Int32],
               la=Layout.ColMajor[GK.Int32], lb=Layout.ColMajor[GK.Int32], lc=Layout.ColMajor[GK.Int32],
               ld=Layout.ColMajor[GK.Int32], alpha=2, beta=3, block_shape=(64, 64, 32))
    assert np.array_equal(GK.to_numpy(d), want["int32_wrap/D"])


def test_golden_tropical(golden):
    cases, want = golden
    cs = cases["tropical"]
    A, B, Cm = cs["A"], cs["B"], cs["C"]
    M, K = A.shape; N = B.shape[1]
    c = dev(Cm); d = GK.cuarray(GK.Float32, M, N)
    run_matmul(dev(A), dev(B), c, d, M=M, N=N, K=K,
               op=Operator.TropicalFPUOp[8, 16, 2, 4, 8, 1, GK.Float32, GK.Float32],
               la=Layout.ColMajor[GK.Float32], lb=Layout.ColMajor[GK.Float32], lc=Layout.ColMajor[GK.Float32],
               ld=Layout.ColMajor[GK.Float32], block_shape=(64, 64, 32))
    assert np.array_equal(GK.to_numpy(d), want["tropical/D"])


# ------------------------------------------------------------------------------------------------
# replay of test/blas.jl: matmatmul! with all transposes, unaligned sizes, random alpha/beta
# ------------------------------------------------------------------------------------------------
BLAS_TYPES = [("Float16", "Float32", True, 128), ("Float16", "Float16", True, 256), ("Float32", "Float32", False, 128)]


@pytest.mark.parametrize("ab,cd,wmma,min_dim", BLAS_TYPES)
@pytest.mark.parametrize("ta,tb", [("N", "N"), ("N", "T"), ("T", "N"), ("T", "T")])
def test_blas_matmatmul(ab, cd, wmma, min_dim, ta, tb):
    rng = np.random.default_rng(hash((ab, cd, ta, tb)) % 2 ** 32)
    AB, CD = getattr(GK, ab), getattr(GK, cd)
    # all 27 combinations of test/blas.jl:19-21
    dims = (10, min_dim, 1000)
    for (M, N, K) in itertools.product(dims, dims, dims):
        alpha, beta = float(rng.random()), float(rng.random())
        A = (rng.random((K, M) if ta == "T" else (M, K)) / math.sqrt(K)).astype(AB.np_dtype)
        B = (rng.random((N, K) if tb == "T" else (K, N)) / math.sqrt(K)).astype(AB.np_dtype)
        Cm = rng.random((M, N)).astype(CD.np_dtype)
        c = dev(Cm)
        a_d, b_d = dev(A), dev(B)
        out = GK.matmatmul_(c, ta, tb, a_d, b_d, alpha, beta, wmma=wmma)
        torch.cuda.synchronize(); GK.poll_status()
        assert out is c
        if wmma:      # every wmma = true case of test/blas.jl runs on the tensor cores, whatever its alignment
            ld = GK.arrays.leading_dimension
            conf, _, kern = GK.create_config(AB, tuple(a_d.shape), (1, ld(a_d)), ta == "T", AB, tuple(b_d.shape), (1, ld(b_d)),
                                             tb == "T", CD, (M, N), (1, ld(c)), alpha == 0, beta == 0, wmma)
            assert GK.query(conf, a_d, b_d, c, c, kernel=kern).kernel == 1, (M, N, K)
        want = O.gemm(A, B, Cm, alpha, beta, ta == "T", tb == "T")
        got = GK.to_numpy(c)
        assert O.isapprox_normwise(want, got, cd if cd == "Float16" else ab), (M, N, K, O.normwise_error(got, want))
        assert O.normwise_error(got, want) <= (TOL_FPU if ab == "Float32" else (2e-3 if cd == "Float16" else TOL_TENSOR))


@pytest.mark.parametrize("ab", ["Float16", "BFloat16"])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_unaligned_operands_stay_on_the_tensor_cores(ab, ta, tb):
    """Leading dimensions and base addresses that are not multiples of 16 bytes (the reference's
    bounds-checked ColMajor / RowMajor layouts, src/layout.jl:111-184, which its WMMA operator runs on
    the sizes of test/blas.jl:19-21): the tcgen05 kernel runs them with ordinary loads in its producer
    warps instead of TMA.  The plan must say tensor cores; small-integer inputs make the result exact."""
    ET = getattr(GK, ab)
    rng = np.random.default_rng(100 + 2 * ta + tb)
    for (M, N, K) in [(10, 10, 10), (10, 128, 1000), (1000, 10, 128), (130, 70, 10), (333, 257, 75), (129, 1, 2050)]:
        A = rng.integers(-2, 3, (K, M) if ta else (M, K)).astype(np.float32)
        B = rng.integers(-2, 3, (N, K) if tb else (K, N)).astype(np.float32)
        Cm = rng.integers(-4, 5, (M, N)).astype(np.float32)

        def odd_storage(x):
            # column-major with a leading dimension of rows + 3 elements, starting one element into the buffer
            r, c = x.shape
            store = torch.zeros(c * (r + 3) + 1, dtype=ET.torch_dtype(), device="cuda")
            view = store[1:].view(c, r + 3)[:, :r].t()
            view.copy_(torch.from_numpy(x).to(ET.torch_dtype()))
            return view
        a, b = odd_storage(A), odd_storage(B)
        assert a.data_ptr() % 16 != 0
        c = dev(Cm)
        conf = GK.get_config(gemm_shape=(M, N, K), operator=Operator.TCGen05Operator[ET, GK.Float32],
                             global_a_layout=(Layout.RowMajor if ta else Layout.ColMajor)[ET],
                             global_b_layout=(Layout.RowMajor if tb else Layout.ColMajor)[ET],
                             global_c_layout=Layout.ColMajor[GK.Float32], global_d_layout=Layout.ColMajor[GK.Float32],
                             is_a_col_major=not ta, is_b_col_major=not tb)
        plan = GK.query(conf, a, b, c, c)
        assert plan.kernel == 1 and plan.cluster == 1, (M, N, K, plan.kernel)
        GK.matmul(conf, a, b, c, c, transform_shared_to_regs_a=Transform.Elementwise(Transform.Scale(2.0)))
        torch.cuda.synchronize(); GK.poll_status()
        want = O.gemm(A, B, Cm, 2.0, 1.0, bool(ta), bool(tb))
        assert np.array_equal(GK.to_numpy(c), want), (M, N, K)


def test_mul_with_transposed_views():
    rng = np.random.default_rng(5)
    A = rng.random((256, 384)).astype(np.float16); Bt = rng.random((128, 384)).astype(np.float16)
    c = GK.cuarray(GK.Float32, 256, 128)
    GK.mul_(c, dev(A), dev(Bt).T)          # C = A * Bt'
    torch.cuda.synchronize()
    assert O.normwise_error(GK.to_numpy(c), O.gemm(A, Bt, trans_b=True)) <= TOL_TENSOR


# ------------------------------------------------------------------------------------------------
# benchmark configurations at full size
# ------------------------------------------------------------------------------------------------
def test_config1_fp16_2048_against_cpu_product():
    """Configuration 1: A, B Float16 ~ U[0,1), 2048^3, alpha = 1, beta = 0, checked against the CPU
    product of the Float32-promoted inputs."""
    A, B = O.inputs_fp16_uniform01(1, 2048, 2048, 2048)
    c = GK.cuarray(GK.Float32, 2048, 2048); c.zero_()
    GK.mul_(c, dev(A), dev(B))
    torch.cuda.synchronize(); GK.poll_status()
    want = O.gemm(A, B)
    got = GK.to_numpy(c)
    assert O.normwise_error(got, want) <= TOL_TENSOR
    assert O.isapprox_elementwise(want, got, "Float16")


def test_metric_shape_8192_sampled_rows_and_linearity():
    """8192^3 FP16 -> FP32 (the headline shape).  A full CPU product would take minutes, so the
    result is checked on 48 sampled rows against the oracle, and through linearity:
    (A1 + A2) B = A1 B + A2 B holds exactly in exact arithmetic and to rounding here."""
    n = 8192
    A, B = O.inputs_fp16_uniform01(0, n, n, n)
    a, b = dev(A), dev(B)
    c = GK.cuarray(GK.Float32, n, n)
    GK.mul_(c, a, b)
    torch.cuda.synchronize(); GK.poll_status()
    rows = np.random.default_rng(0).choice(n, 48, replace=False)
    want = A[rows].astype(np.float32) @ B.astype(np.float32)
    got = c[torch.from_numpy(rows).cuda()].cpu().numpy()
    assert O.normwise_error(got, want) <= TOL_TENSOR
    # 2*A is exact in Float16 here (values in [0, 1)), so every product and partial sum doubles
    # exactly: the result must be 2*C bit for bit.
    c2 = GK.cuarray(GK.Float32, n, n)
    GK.mul_(c2, dev((A * np.float16(2)).astype(np.float16)), b)
    torch.cuda.synchronize()
    assert torch.equal(c2, c * 2)
    # additivity: split A exactly into a coarse part and a remainder, A = A1 + A2
    A1 = (A.view(np.uint16) & np.uint16(0xFFE0)).view(np.float16)
    A2 = (A.astype(np.float32) - A1.astype(np.float32)).astype(np.float16)
    assert np.array_equal(A1.astype(np.float32) + A2.astype(np.float32), A.astype(np.float32))
    c3 = GK.cuarray(GK.Float32, n, n)
    GK.mul_(c2, dev(A1), b)
    GK.mul_(c3, dev(A2), b)
    torch.cuda.synchronize(); GK.poll_status()
    assert ((c2 + c3) - c).norm().item() / c.norm().item() <= 1e-4   # FP32 accumulation noise over K = 8192


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("cg,bn", [(1, 128), (2, 256), (1, 256), (2, 128), (2, 512)])
def test_tile_shapes_and_transposes_exact(ta, tb, cg, bn):
    """Small-integer inputs make the FP16 -> FP32 product exact, so any layout / descriptor slip
    shows as a hard mismatch rather than as noise."""
    rng = np.random.default_rng(cg * 1000 + bn + ta * 2 + tb)
    M, N, K = 640, 520, 392
    A = rng.integers(-2, 3, (K, M) if ta else (M, K)).astype(np.float16)
    B = rng.integers(-2, 3, (N, K) if tb else (K, N)).astype(np.float16)
    d = GK.cuarray(GK.Float32, M, N)
    la = (Layout.RowMajor if ta else Layout.ColMajor)[GK.Float16]
    lb = (Layout.RowMajor if tb else Layout.ColMajor)[GK.Float16]
    run_matmul(dev(A), dev(B), None, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[GK.Float16, GK.Float32],
               la=la, lb=lb, lc=Layout.Zero[GK.Float32], ld=Layout.ColMajor[GK.Float32],
               block_shape=(128, 128, 64), cta_group=cg, tile_n=bn)
    assert np.array_equal(GK.to_numpy(d), O.gemm(A, B, trans_a=bool(ta), trans_b=bool(tb)))


@pytest.mark.parametrize("ta,tb,K", [(0, 0, 512), (1, 0, 640), (0, 1, 1088), (1, 1, 576)])
def test_wide_tiles_skewed_schedule_exact(ta, tb, K):
    """256 x 512 tiles with K of at least two pipeline rings run the skewed schedule: the two 256-column blocks
    of a tile start and finish half a ring apart, each behind its own accumulator barrier.  190 tiles on 74
    CTA pairs (two or three tiles per pair, so the barriers change phase), a ragged last tile column, small
    integers: any slip in the order of MMAs, commits or epilogue passes is a hard mismatch.  Twice, on the
    same operands, to catch state left behind by the first launch."""
    M, N = 2560, 9504
    rng = np.random.default_rng(K + ta * 2 + tb)
    A = rng.integers(-2, 3, (K, M) if ta else (M, K)).astype(np.float16)
    B = rng.integers(-2, 3, (N, K) if tb else (K, N)).astype(np.float16)
    la = (Layout.RowMajor if ta else Layout.ColMajor)[GK.Float16]
    lb = (Layout.RowMajor if tb else Layout.ColMajor)[GK.Float16]
    want = O.gemm(A, B, trans_a=bool(ta), trans_b=bool(tb))
    a, b = dev(A), dev(B)
    for _ in range(2):
        d = GK.cuarray(GK.Float32, M, N); d.fill_(-7.0)
        conf = run_matmul(a, b, None, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                          la=la, lb=lb, lc=Layout.Zero[GK.Float32], ld=Layout.ColMajor[GK.Float32],
                          block_shape=(128, 128, 64), cta_group=2, tile_n=512)
        plan = GK.query(conf, a, b, None, d)
        assert plan.tile_n == 512 and plan.tmem_columns == 512 and K // 64 >= 2 * plan.stages
        assert np.array_equal(GK.to_numpy(d), want)


@pytest.mark.parametrize("swizzle", [CTASwizzle.Identity(), CTASwizzle.HorizontallyTiled[2], CTASwizzle.HorizontallyTiled[8],
                                     CTASwizzle.VerticallyTiled[3], CTASwizzle.LebesgueCurve()])
@pytest.mark.parametrize("M,N", [(2048, 2048), (1024, 4096), (1400, 900)])
def test_every_cta_swizzle_visits_every_tile(swizzle, M, N):
    """The raster only changes the order of tiles: results are identical, and exact on integers.
    2048 x 2048 and 1024 x 4096 are power-of-two tile grids (the Z-order walk), 1400 x 900 is not."""
    rng = np.random.default_rng(M + N)
    K = 192
    A = rng.integers(-2, 3, (M, K)).astype(np.float16); B = rng.integers(-2, 3, (K, N)).astype(np.float16)
    d = GK.cuarray(GK.Float32, M, N); d.fill_(-1.0)
    run_matmul(dev(A), dev(B), None, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[GK.Float16, GK.Float32],
               la=Layout.ColMajor[GK.Float16], lb=Layout.ColMajor[GK.Float16], lc=Layout.Zero[GK.Float32],
               ld=Layout.ColMajor[GK.Float32], block_shape=(128, 128, 64), cta_swizzle=swizzle, tile_n=128, cta_group=1)
    assert np.array_equal(GK.to_numpy(d), A.astype(np.float32) @ B.astype(np.float32))


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_tf32(ta, tb):
    rng = np.random.default_rng(9 + ta * 2 + tb)
    M, N, K = 384, 256, 520
    A = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    B = rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    d = GK.cuarray(GK.Float32, M, N)
    la = (Layout.RowMajor if ta else Layout.ColMajor)[GK.Float32]
    lb = (Layout.RowMajor if tb else Layout.ColMajor)[GK.Float32]
    run_matmul(dev(A), dev(B), None, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[Operator.TF32, GK.Float32],
               la=la, lb=lb, lc=Layout.Zero[GK.Float32], ld=Layout.ColMajor[GK.Float32], block_shape=(128, 128, 32))
    got = GK.to_numpy(d)
    assert O.normwise_error(got, O.gemm64(A, B, trans_a=bool(ta), trans_b=bool(tb))) <= TOL_TENSOR
    # and it is what TF32 inputs give: tighter against the truncated-input product
    assert O.normwise_error(got, O.gemm64(O.tf32_truncate(A), O.tf32_truncate(B), trans_a=bool(ta), trans_b=bool(tb))) <= 2e-5


def test_config3_planar_complex_4096_sampled():
    """Configuration 3 at full size (4096^3 planar complex FP16 -> Complex{F32}): sampled rows."""
    n = 4096
    A, B = O.inputs_planar_fp16(3, n, n, n)
    d = GK.cuarray(GK.Float32, n, n, 2)
    run_matmul(planar(A), planar(B), None, d, M=n, N=n, K=n, op=Operator.WMMAComplexOp[16, 16, 16, GK.Float16, GK.Float32],
               la=Layout.SplitColMajor[GK.Float16], lb=Layout.SplitColMajor[GK.Float16],
               lc=Layout.Zero[GK.Float32], ld=Layout.SplitColMajor[GK.Float32], block_shape=(64, 64, 32))
    rows = np.random.default_rng(1).choice(n, 32, replace=False)
    re, im = O.complex_gemm(A[0][rows], A[1][rows], B[0], B[1])
    got = d[torch.from_numpy(rows).cuda()].cpu().numpy()      # (32, n, 2)
    assert O.normwise_error(got[..., 0], re) <= TOL_TENSOR and O.normwise_error(got[..., 1], im) <= TOL_TENSOR


@pytest.mark.parametrize("opcls,ref", [(Operator.WMMAComplexOp, "complex"), (Operator.WMMADualOp, "dual")])
def test_planar_complex_dual_single_accumulator_stage(opcls, ref):
    """tile_n = 256 with two accumulator planes fills all 512 TMEM columns: the single-stage
    schedule (epilogue not overlapped) must give the same numbers; several tiles per CTA pair."""
    M, N, K = 4096, 2560, 256
    rng = np.random.default_rng(77)
    A = rng.integers(-2, 3, (2, M, K)).astype(np.float16); B = rng.integers(-2, 3, (2, K, N)).astype(np.float16)
    d = GK.cuarray(GK.Float32, M, N, 2)
    conf = run_matmul(planar(A), planar(B), None, d, M=M, N=N, K=K, op=opcls[16, 16, 16, GK.Float16, GK.Float32],
                      la=Layout.SplitColMajor[GK.Float16], lb=Layout.SplitColMajor[GK.Float16],
                      lc=Layout.Zero[GK.Float32], ld=Layout.SplitColMajor[GK.Float32], block_shape=(64, 64, 32),
                      tile_n=256, cta_group=2)
    plan = GK.query(conf, planar(A), planar(B), None, d)
    assert plan.tile_n == 256 and plan.tmem_columns == 512
    p0, p1 = (O.complex_gemm if ref == "complex" else O.dual_gemm)(A[0], A[1], B[0], B[1])
    got = GK.to_numpy(d)
    assert np.array_equal(got[..., 0], p0) and np.array_equal(got[..., 1], p1)     # small integers: exact


# ------------------------------------------------------------------------------------------------
# edge cases and error behaviour
# ------------------------------------------------------------------------------------------------
def test_beta_with_aliased_c_and_d_and_fp16_output():
    rng = np.random.default_rng(21)
    M, N, K = 256, 136, 72
    A = rng.random((M, K)).astype(np.float16); B = rng.random((K, N)).astype(np.float16)
    Cm = rng.random((M, N)).astype(np.float16)
    c = dev(Cm)
    GK.matmatmul_(c, "N", "N", dev(A), dev(B), 2.0, 3.0, wmma=True)
    torch.cuda.synchronize()
    want = O.gemm(A, B, Cm, 2.0, 3.0)
    assert O.isapprox_elementwise(want, GK.to_numpy(c), "Float16")


def test_fp32_fma_rate_measurement_is_plausible():
    """gk_measure_fp32_fma: between half of and a little above the nominal 148 x 128 x 2 x clock."""
    import ctypes as C
    from gemmkernels_b200 import _lib as L
    out = C.c_double(0.0)
    assert L.lib.gk_measure_fp32_fma(GK.handle(), C.byref(out), C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    props = torch.cuda.get_device_properties(0)
    nominal = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    assert 0.5 * nominal < out.value < 1.1 * nominal, out.value


def test_bound_matmul_replays_the_same_gemm():
    """GK.bind lowers once; each call of the object enqueues the same GEMM (here in place: D = A*B + D)."""
    rng = np.random.default_rng(22)
    M, N, K = 384, 320, 192
    A = rng.integers(-2, 3, (M, K)).astype(np.float16); B = rng.integers(-2, 3, (K, N)).astype(np.float16)
    d = dev(np.zeros((M, N), dtype=np.float32))
    conf = GK.get_config(gemm_shape=(M, N, K), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                         global_a_layout=Layout.ColMajor[GK.Float16], global_c_layout=Layout.ColMajor[GK.Float32])
    launch = GK.bind(conf, dev(A), dev(B), d, d)
    for _ in range(3):
        launch()
    torch.cuda.synchronize(); GK.poll_status()
    assert np.array_equal(GK.to_numpy(d), 3 * (A.astype(np.float32) @ B.astype(np.float32)))


@pytest.mark.parametrize("cd", ["Float32", "Float16", "BFloat16"])
@pytest.mark.parametrize("bias_axis,act", [(None, None), ("col", Transform.GELU()), ("row", Transform.ReLU())])
def test_epilogue_variants_full_and_ragged_chunks(cd, bias_axis, act):
    """alpha*A*B + beta*C with C and D of one type, N not a multiple of 32: full chunks take the
    type-specialised epilogue, the last chunk the element-wise one; both must agree with the oracle."""
    rng = np.random.default_rng(23)
    M, N, K = 300, 1000, 136
    CD = getattr(GK, cd)
    AB = GK.BFloat16 if cd == "BFloat16" else GK.Float16         # BFloat16 results come from BFloat16 operands
    A = (rng.integers(-8, 9, (M, K)) / 16).astype(np.float32); B = (rng.integers(-8, 9, (K, N)) / 16).astype(np.float32)
    Cm = (rng.random((M, N)) - 0.5).astype(np.float32)
    c = dev(Cm, CD); Cq = GK.to_numpy(c).astype(np.float32)
    d = GK.cuarray(CD, M, N)
    bias = (rng.random(M if bias_axis == "row" else N) - 0.5).astype(np.float32) if bias_axis else None
    epi = Epilogue.Bias(torch.from_numpy(bias).cuda(), axis=bias_axis) if bias_axis else None
    run_matmul(dev(A, AB), dev(B, AB), c, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[AB, GK.Float32],
               la=Layout.ColMajor[AB], lb=Layout.ColMajor[AB], lc=Layout.ColMajor[CD], ld=Layout.ColMajor[CD],
               alpha=1.5, beta=0.5, epilogue=epi, act=act)
    want = 1.5 * (A.astype(np.float32) @ B.astype(np.float32)) + 0.5 * Cq
    want = O.epilogue(want, bias, bias_axis or "col", {Transform.ReLU: "relu", Transform.GELU: "gelu"}.get(type(act)))
    tol = {"Float32": 1e-5, "Float16": 1e-3, "BFloat16": 8e-3}[cd]
    assert O.normwise_error(GK.to_numpy(d).astype(np.float32), want) <= tol


def test_leading_dimension_larger_than_rows():
    rng = np.random.default_rng(22)
    M, N, K, ld = 200, 96, 64, 264
    big = torch.zeros(K, ld, dtype=torch.float16, device="cuda").T      # (ld, K) column-major
    A = rng.random((M, K)).astype(np.float16)
    big[:M] = torch.from_numpy(A).cuda()
    a = big[:M]                                                        # view with ld = 264
    assert a.stride(1) == ld
    B = rng.random((K, N)).astype(np.float16)
    c = GK.cuarray(GK.Float32, M, N)
    GK.mul_(c, a, dev(B))
    torch.cuda.synchronize()
    assert O.normwise_error(GK.to_numpy(c), O.gemm(A, B)) <= TOL_TENSOR


def test_alpha_zero_and_k_zero_reduce_to_beta_c():
    rng = np.random.default_rng(23)
    Cm = rng.random((64, 48)).astype(np.float32)
    A = rng.random((64, 32)).astype(np.float16); B = rng.random((32, 48)).astype(np.float16)
    c = dev(Cm)
    GK.matmatmul_(c, "N", "N", dev(A), dev(B), 0.0, 0.5, wmma=True)
    torch.cuda.synchronize()
    assert np.allclose(GK.to_numpy(c), 0.5 * Cm, rtol=1e-6)


@pytest.mark.parametrize("M,N,K", [(0, 8, 8), (8, 0, 8), (1, 1, 1), (1, 7, 3), (33, 1, 129), (2, 300, 1)])
def test_empty_and_tiny_products(M, N, K):
    """Empty outputs are a no-op; sizes far below a tile go through whichever kernel takes them."""
    rng = np.random.default_rng(M * 100 + N * 10 + K)
    A = rng.integers(-3, 4, (M, K)).astype(np.float16); B = rng.integers(-3, 4, (K, N)).astype(np.float16)
    Cm = rng.integers(-3, 4, (M, N)).astype(np.float32)
    c = dev(Cm) if M * N else GK.cuarray(GK.Float32, M, N)
    out = GK.matmatmul_(c, "N", "N", dev(A) if M * K else GK.cuarray(GK.Float16, M, K),
                        dev(B) if K * N else GK.cuarray(GK.Float16, K, N), 2.0, 1.0)
    torch.cuda.synchronize(); GK.poll_status()
    assert out is c and tuple(c.shape) == (M, N)
    if M * N:
        assert np.array_equal(GK.to_numpy(c), 2.0 * (A.astype(np.float32) @ B.astype(np.float32)) + Cm)


@pytest.mark.parametrize("M,N,K,ta,cd,beta,bias_axis,act", [
    (256, 256, 16384, False, "Float32", 0.0, None, None),
    (384, 520, 8192, False, "Float32", 0.5, "col", Transform.ReLU()),
    (130, 264, 4096, True, "Float16", 1.0, "row", None),    # M not a multiple of 4 (A stored transposed): scalar reduction pass
])
def test_split_k_for_few_tiles_and_long_k(M, N, K, ta, cd, beta, bias_axis, act):
    """Few output tiles, long K: the product is cut along K over the idle SMs (partial sums in a
    workspace the Python layer allocates from gk_gemm_query's figure) and reduced in a second pass."""
    rng = np.random.default_rng(M + K)
    CD = getattr(GK, cd)
    A = rng.integers(-2, 3, (M, K)).astype(np.float16); B = rng.integers(-2, 3, (K, N)).astype(np.float16)
    Cm = rng.integers(-8, 9, (M, N)).astype(np.float32)
    bias = rng.integers(-4, 5, M if bias_axis == "row" else N).astype(np.float32) if bias_axis else None
    c = dev(Cm, CD) if beta else None
    d = GK.cuarray(CD, M, N)
    epi = Epilogue.Bias(torch.from_numpy(bias).cuda(), axis=bias_axis) if bias_axis else None
    a_dev = dev(A.T.copy() if ta else A)
    conf = run_matmul(a_dev, dev(B), c, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                      la=(Layout.RowMajor if ta else Layout.ColMajor)[GK.Float16], lb=Layout.ColMajor[GK.Float16],
                      lc=(Layout.ColMajor if beta else Layout.Zero)[CD], ld=Layout.ColMajor[CD],
                      beta=beta if beta else 1.0, epilogue=epi, act=act)
    plan = GK.query(conf, a_dev, dev(B), c, d, epilogue=epi)
    assert plan.kernel == 1 and plan.workspace_bytes >= 2 * 4 * M * N          # at least two partial planes
    want = A.astype(np.float64) @ B.astype(np.float64)
    if beta:
        want = want + beta * Cm
    want = O.epilogue(want, bias, bias_axis or "col", "relu" if act is not None else None)
    got = GK.to_numpy(d).astype(np.float64)
    if cd == "Float32":
        assert np.array_equal(got, want)                   # small integers: exact whatever the summation order
    else:
        assert O.normwise_error(got, want) <= 1e-3
    # without a workspace the same call runs unsplit and gives the same numbers
    d2 = GK.cuarray(CD, M, N)
    hooks = {}
    if beta not in (0.0, 1.0):
        hooks["shared_to_regs_c"] = Transform.Elementwise(Transform.Scale(beta))
    if act is not None:
        hooks["shared_to_global_d"] = Transform.Elementwise(act)
    desc, epi_desc, (pa, pb, pc, _) = GK.lower(conf, a_dev, dev(B), c, d2, hooks, epi or Epilogue.Default(), Kernel.matmul_singlestage)
    B_d = dev(B)
    assert L.lib.gk_gemm(GK.handle(), C.byref(desc), a_dev.data_ptr(), B_d.data_ptr(), pc, d2.data_ptr(), C.byref(epi_desc), None, 0,
                         C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize(); GK.poll_status()
    assert torch.equal(d2, d) if cd == "Float32" else O.normwise_error(GK.to_numpy(d2).astype(np.float64), want) <= 1e-3


def test_split_k_never_writes_past_a_small_workspace():
    """A workspace smaller than the partial sums need is used for as many K-runs as it holds (or not
    at all); a canary directly behind it must survive, and the result is the same product."""
    M, N, K = 256, 256, 16384
    rng = np.random.default_rng(9)
    A = rng.integers(-2, 3, (M, K)).astype(np.float16); B = rng.integers(-2, 3, (K, N)).astype(np.float16)
    a, b = dev(A), dev(B)
    conf = GK.get_config(gemm_shape=(M, N, K), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                         global_a_layout=Layout.ColMajor[GK.Float16], global_c_layout=Layout.Zero[GK.Float32],
                         global_d_layout=Layout.ColMajor[GK.Float32])
    want = O.gemm(A, B)
    full = GK.query(conf, a, b, None, GK.cuarray(GK.Float32, M, N)).workspace_bytes
    assert full >= 2 * M * N * 4
    for ws_bytes in (full, 3 * M * N * 4, M * N * 4 + 4096, 4096):
        buf = torch.zeros(ws_bytes + 4096, dtype=torch.uint8, device="cuda")
        buf[ws_bytes:] = 0xA5
        d = GK.cuarray(GK.Float32, M, N)
        desc, epi_desc, (pa, pb, pc, pd) = GK.lower(conf, a, b, None, d, {}, Epilogue.Default(), Kernel.matmul_singlestage)
        st = L.lib.gk_gemm(GK.handle(), C.byref(desc), pa, pb, pc, pd, C.byref(epi_desc), buf.data_ptr(), ws_bytes,
                           C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert st == L.GK_OK, L.last_error()
        torch.cuda.synchronize(); GK.poll_status()
        assert torch.all(buf[ws_bytes:] == 0xA5), ws_bytes
        assert np.array_equal(GK.to_numpy(d), want), ws_bytes


@pytest.mark.parametrize("ab,op", [("Float16", "tc"), ("Float32", "fpu"), ("Int32", "simt")])
@pytest.mark.parametrize("share_b", [False, True])
def test_strided_batched_products(ab, op, share_b):
    """`batch` products in one call: tensor cores walk (product, tile) pairs in one launch, the SIMT
    families launch once per product.  Operands padded between the products; B optionally shared."""
    M, N, K, nb = 384, 320, 192, 5
    if op == "fpu":
        M, N, K = 256, 128, 64
    rng = np.random.default_rng(11)
    ET = getattr(GK, ab); CD = GK.Int32 if ab == "Int32" else GK.Float32
    A = rng.integers(-3, 4, (nb, M, K)).astype(ET.np_dtype)
    B = rng.integers(-3, 4, (1 if share_b else nb, K, N)).astype(ET.np_dtype)
    Cm = rng.integers(-5, 6, (nb, M, N)).astype(CD.np_dtype)

    def batched(x, pad):
        # (nb, r, c) numpy -> device (r, c, nb) with `pad` unused elements between the matrices
        nbx, r, c = x.shape
        store = torch.zeros(nbx, r * c + pad, dtype=torch.from_numpy(x[:1]).dtype, device="cuda")
        store[:, : r * c] = torch.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 1))).reshape(nbx, r * c).cuda()
        return store[:, : r * c].view(nbx, c, r).permute(2, 1, 0), store

    a, _ = batched(A, 64)
    b, _ = batched(B, 128)
    if share_b:
        b = b[:, :, 0]
    c, _ = batched(Cm, 32)
    d, d_store = batched(np.zeros_like(Cm), 96)
    if op == "tc":
        oper = Operator.TCGen05Operator[ET, CD]
    else:
        oper = Operator.FPUOp[8, 8, 1, 4, 8, 1, ET, CD]
    conf = GK.get_config(gemm_shape=(M, N, K), operator=oper, global_a_layout=Layout.ColMajor[ET],
                         global_b_layout=Layout.ColMajor[ET], global_c_layout=Layout.ColMajor[CD],
                         global_d_layout=Layout.ColMajor[CD], **({"block_shape": (64, 64, 32)} if op != "tc" else {}))
    GK.matmul_batched(conf, a, b, c, d, transform_shared_to_regs_a=Transform.Elementwise(Transform.Scale(2)))
    torch.cuda.synchronize(); GK.poll_status()
    got = GK.to_numpy(d)
    for i in range(nb):
        Bi = B[0 if share_b else i]
        if ab == "Int32":
            want = O.integer_gemm(A[i], Bi, Cm[i], 2, 1)
        else:
            want = O.gemm(A[i], Bi, Cm[i], 2.0, 1.0)
        assert np.array_equal(got[:, :, i], want), i        # small integers: exact
    # the padding between the outputs is untouched
    assert torch.all(d_store[:, M * N:] == 0)


@pytest.mark.parametrize("shape,split_tiles,parts", [((2560, 2304, 1024), 64, 4), ((384, 512, 1056), 12, 8)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (1, 1)])
def test_fpu_tail_split_matches_the_unsplit_product(ta, tb, shape, split_tiles, parts):
    """FFMA kernel, 360 tiles on 296 CTA slots: given a workspace, the 64 tiles of the last round are cut
    along K in four parts that run side by side and a second pass adds them and applies beta, bias and
    ReLU.  A grid of 12 tiles, too small for the GPU, has every tile cut in eight parts (66 k-tiles: the
    last part is shorter).  Same numbers as the unsplit launch (small integers: exact), nothing written
    past the workspace."""
    M, N, K = shape
    rng = np.random.default_rng(31 + ta + 2 * tb)
    A = rng.integers(-2, 3, (K, M) if ta else (M, K)).astype(np.float32)
    B = rng.integers(-2, 3, (N, K) if tb else (K, N)).astype(np.float32)
    Cm = rng.integers(-4, 5, (M, N)).astype(np.float32); bias = rng.integers(-3, 4, N).astype(np.float32)
    a, b, c = dev(A), dev(B), dev(Cm)
    la = (Layout.UnsafeAlignedRowMajor if ta else Layout.UnsafeAlignedColMajor)[GK.Float32]
    lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[GK.Float32]
    conf = GK.get_config(gemm_shape=(M, N, K), operator=Operator.FPUOp[8, 8, 1, 4, 8, 1, GK.Float32, GK.Float32],
                         global_a_layout=la, global_b_layout=lb, global_c_layout=Layout.UnsafeAlignedColMajor[GK.Float32],
                         global_d_layout=Layout.UnsafeAlignedColMajor[GK.Float32], is_a_col_major=not ta, is_b_col_major=not tb)
    epi = Epilogue.Bias(dev(bias), axis="col")
    kw = dict(epilogue=epi, transform_shared_to_global_d=Transform.Elementwise(Transform.ReLU()),
              transform_shared_to_regs_a=Transform.Elementwise(Transform.Scale(2.0)))
    plan = GK.query(conf, a, b, c, GK.cuarray(GK.Float32, M, N), **kw)
    assert plan.kernel == 2 and plan.workspace_bytes == split_tiles * parts * 128 * 128 * 4
    want = np.maximum(2.0 * ((A.T if ta else A) @ (B.T if tb else B)) + Cm + bias[None, :], 0)
    d_split = GK.cuarray(GK.Float32, M, N)
    ws = torch.zeros(plan.workspace_bytes + 4096, dtype=torch.uint8, device="cuda"); ws[plan.workspace_bytes:] = 0x5A
    GK.matmul(conf, a, b, c, d_split, workspace=ws[:plan.workspace_bytes], **kw)
    torch.cuda.synchronize(); GK.poll_status()
    assert np.array_equal(GK.to_numpy(d_split), want)
    assert torch.all(ws[plan.workspace_bytes:] == 0x5A) and ws[:plan.workspace_bytes].any()      # used, and not overrun
    d_plain = GK.cuarray(GK.Float32, M, N)
    small = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")                                 # too small: unsplit
    GK.matmul(conf, a, b, c, d_plain, workspace=small, **kw)
    torch.cuda.synchronize(); GK.poll_status()
    assert torch.equal(d_plain, d_split)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_fp64_fast_path_matches_float64_numpy(ta, tb):
    """Float64 FPU operator on tile-multiple, aligned shapes: the FP64 kernel (family 2 in the plan), all four
    transposes, alpha, beta, per-column bias and ReLU fused.  Small integers make the sums exact; a second
    product with random operands is held to 1e-12 normwise against numpy's float64 product."""
    M, N, K = 1536, 1280, 224          # 120 tiles: the fast path wants three quarters of a round
    rng = np.random.default_rng(41 + ta + 2 * tb)
    la = (Layout.UnsafeAlignedRowMajor if ta else Layout.UnsafeAlignedColMajor)[GK.Float64]
    lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[GK.Float64]
    op = Operator.FPUOp[8, 8, 1, 4, 8, 1, GK.Float64, GK.Float64]
    for exact in (True, False):
        if exact:
            A = rng.integers(-3, 4, (K, M) if ta else (M, K)).astype(np.float64)
            B = rng.integers(-3, 4, (N, K) if tb else (K, N)).astype(np.float64)
            Cm = rng.integers(-5, 6, (M, N)).astype(np.float64); bias = rng.integers(-3, 4, N).astype(np.float32)
        else:
            A = rng.standard_normal((K, M) if ta else (M, K)); B = rng.standard_normal((N, K) if tb else (K, N))
            Cm = rng.standard_normal((M, N)); bias = rng.standard_normal(N).astype(np.float32)
        a, b, c, d = dev(A), dev(B), dev(Cm), GK.cuarray(GK.Float64, M, N)
        conf = run_matmul(a, b, c, d, M=M, N=N, K=K, op=op, la=la, lb=lb, lc=Layout.UnsafeAlignedColMajor[GK.Float64],
                          ld=Layout.UnsafeAlignedColMajor[GK.Float64], alpha=2.0, beta=3.0,
                          epilogue=Epilogue.Bias(dev(bias), axis="col"), act=Transform.ReLU(), block_shape=(128, 128, 32))
        plan = GK.query(conf, a, b, c, d, epilogue=Epilogue.Bias(dev(bias), axis="col"),
                        transform_shared_to_global_d=Transform.Elementwise(Transform.ReLU()))
        assert plan.kernel == 2 and plan.tile_m == 128 and plan.block == 256
        want = np.maximum(2.0 * ((A.T if ta else A) @ (B.T if tb else B)) + 3.0 * Cm + bias[None, :].astype(np.float64), 0)
        got = GK.to_numpy(d)
        if exact:
            assert np.array_equal(got, want)
        else:
            assert O.normwise_error(got, want) <= 1e-12


@pytest.mark.parametrize("axis,act,beta", [("row", Transform.GELU(), 1.0), ("row", None, 0.0), (None, Transform.ReLU(), 0.5)])
def test_fp64_fast_path_epilogue_variants(axis, act, beta):
    """The FP64 kernel's other epilogue paths: per-row bias, GELU, no bias, beta = 0 (C not read) — against float64
    numpy (erf from math), 1e-12 normwise."""
    import math
    M, N, K = 1536, 1280, 96
    rng = np.random.default_rng(5)
    A = rng.standard_normal((K, M)); B = rng.standard_normal((K, N)); Cm = rng.standard_normal((M, N))
    bias = rng.standard_normal(M).astype(np.float32)
    a, b, c, d = dev(A), dev(B), dev(Cm), GK.cuarray(GK.Float64, M, N)
    epi = Epilogue.Bias(dev(bias), axis=axis) if axis else None
    run_matmul(a, b, c if beta != 0.0 else None, d, M=M, N=N, K=K, op=Operator.FPUOp[8, 8, 1, 4, 8, 1, GK.Float64, GK.Float64],
               la=Layout.UnsafeAlignedRowMajor[GK.Float64], lb=Layout.UnsafeAlignedColMajor[GK.Float64],
               lc=(Layout.UnsafeAlignedColMajor if beta != 0.0 else Layout.Zero)[GK.Float64],
               ld=Layout.UnsafeAlignedColMajor[GK.Float64], alpha=1.5, beta=beta if beta != 0.0 else 1.0,
               epilogue=epi, act=act, block_shape=(128, 128, 32))
    want = 1.5 * (A.T @ B) + (beta * Cm if beta != 0.0 else 0.0)
    if axis:
        want = want + bias[:, None].astype(np.float64)
    if isinstance(act, Transform.ReLU):
        want = np.maximum(want, 0)
    elif isinstance(act, Transform.GELU):
        want = 0.5 * want * (1.0 + np.vectorize(math.erf)(want / math.sqrt(2.0)))
    assert O.normwise_error(GK.to_numpy(d), want) <= 1e-12


def test_chained_products_without_host_synchronisation():
    """Y = (A*B)*C with the first product's Float16 output feeding the second, ten chains enqueued back to back:
    the second kernel may start its set-up while the first is still running (programmatic dependent launch) but
    must not read X before the first has finished; every chain must give the exact result."""
    n = 2048
    rng = np.random.default_rng(404)
    A = (rng.random((n, n)) < 1 / 64).astype(np.float16); B = (rng.random((n, n)) < 1 / 64).astype(np.float16)
    Cm = rng.integers(-1, 2, (n, n)).astype(np.float16)
    X = A.astype(np.float32) @ B.astype(np.float32)
    assert X.max() <= 2048                                   # exactly representable in Float16
    want = X @ Cm.astype(np.float32)
    a, b, c = dev(A), dev(B), dev(Cm)
    x = GK.cuarray(GK.Float16, n, n); y = GK.cuarray(GK.Float32, n, n)
    lay16, lay32 = Layout.UnsafeAlignedColMajor[GK.Float16], Layout.UnsafeAlignedColMajor[GK.Float32]
    conf1 = GK.get_config(gemm_shape=(n, n, n), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                          global_a_layout=lay16, global_c_layout=Layout.Zero[GK.Float16], global_d_layout=lay16)
    conf2 = GK.get_config(gemm_shape=(n, n, n), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                          global_a_layout=lay16, global_c_layout=Layout.Zero[GK.Float32], global_d_layout=lay32)
    first, second = GK.bind(conf1, a, b, None, x), GK.bind(conf2, x, c, None, y)
    for i in range(10):
        x.zero_(); y.zero_()                                  # stale data would show
        first(); second()
        if i % 3 == 0:
            torch.cuda.synchronize()
            assert np.array_equal(GK.to_numpy(y), want), i
    torch.cuda.synchronize(); GK.poll_status()
    assert np.array_equal(GK.to_numpy(y), want)


def test_unsupported_combinations_raise_config_error():
    a = GK.cuarray(GK.Float64, 128, 128); d = GK.cuarray(GK.Float64, 128, 128)
    conf = GK.get_config(gemm_shape=(128, 128, 128), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                         global_a_layout=Layout.ColMajor[GK.Float64], global_c_layout=Layout.ColMajor[GK.Float64],
                         block_shape=(128, 128, 64))
    with pytest.raises(GK.ConfigError):
        GK.matmul(conf, a, a, d, d)
    with pytest.raises(GK.DimensionMismatch):
        GK.matmatmul_(GK.cuarray(GK.Float32, 64, 64), "N", "N", GK.cuarray(GK.Float16, 64, 32),
                      GK.cuarray(GK.Float16, 48, 64), 1.0, 0.0)


def test_bounded_wait_reports_timeout_and_context_survives():
    """A wait that nothing will ever satisfy (the producers are told to issue no copies) must run
    out, leave an error status for the host, and leave the context usable."""
    n = 256
    a = torch.ones(n, n, dtype=torch.float16, device="cuda").T
    d = GK.cuarray(GK.Float32, n, n)
    desc = L.GemmDesc(number=0, m=n, n=n, k=n, dtype_a=L.GK_F16, dtype_b=L.GK_F16, dtype_c=L.GK_F32, dtype_d=L.GK_F32,
                      compute=L.GK_F16, op=L.GK_OP_TCGEN05, lda=n, ldb=n, ldc=n, ldd=n, alpha=1.0, cta_group=1, tile_n=128)
    desc.debug = 4                # measurement/test aid: producers skip their copies
    h = GK.handle()
    st = L.lib.gk_gemm(h, C.byref(desc), a.data_ptr(), a.data_ptr(), None, d.data_ptr(), None, None, 0,
                       C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == L.GK_OK
    torch.cuda.synchronize()
    with pytest.raises(GK.DeviceTimeout):
        GK.poll_status()
    GK.poll_status()               # status is cleared by the read
    c = GK.cuarray(GK.Float32, n, n)
    GK.mul_(c, a, a)
    torch.cuda.synchronize(); GK.poll_status()
    assert torch.all(c == n)


# ------------------------------------------------------------------------------------------------
# tensor contraction (GETT)
# ------------------------------------------------------------------------------------------------
def _julia_tensor(x):
    """numpy array -> device tensor with column-major (Julia) strides."""
    return GK.to_cuarray(np.asarray(x))


def test_contraction_golden_extents8_gather_and_any_path(golden):
    """C[a,b,c,d] = sum_{e,f} A[a,e,b,f] B[d,f,c,e] with extents 8 (the committed fixture): too small
    for TMA boxes, so it exercises the gather kernel and its offset tables."""
    cases, want = golden
    A, B = cases["contraction_aebf_dfce"]["A"], cases["contraction_aebf_dfce"]["B"]
    d = GK.cuarray(GK.Float32, 8, 8, 8, 8)
    plan = GK.contract_query(d, "abcd", _julia_tensor(A), "aebf", _julia_tensor(B), "dfce")
    assert plan.kernel == 5 and plan.workspace_bytes == 8 * (3 * 64 + 3 * 64 + 2 * 64)
    GK.contract_(d, "abcd", _julia_tensor(A), "aebf", _julia_tensor(B), "dfce")
    torch.cuda.synchronize(); GK.poll_status()
    assert O.normwise_error(GK.to_numpy(d), want["contraction_aebf_dfce/D"]) <= TOL_TENSOR


@pytest.mark.parametrize("force_gather", [False, True])
def test_config4_contraction_extents32(force_gather):
    """Configuration 4: extents 32 (M = N = K = 1024), A, B Float16 ~ U[-1,1), C Float32, modes
    permuted as written; tensor-core path through 5-D tensor maps, and the gather path."""
    A, B = O.inputs_contraction(4, 32)
    a, b = _julia_tensor(A), _julia_tensor(B)
    d = GK.cuarray(GK.Float32, 32, 32, 32, 32)
    plan = GK.contract_query(d, "abcd", a, "aebf", b, "dfce", force_gather=force_gather)
    assert plan.kernel == (5 if force_gather else 1)
    GK.contract_(d, "abcd", a, "aebf", b, "dfce", force_gather=force_gather)
    torch.cuda.synchronize(); GK.poll_status()
    want = O.contract(A, "aebf", B, "dfce", "abcd")
    assert O.normwise_error(GK.to_numpy(d), want) <= TOL_TENSOR
    # the bound form enqueues the same contraction
    d2 = GK.cuarray(GK.Float32, 32, 32, 32, 32)
    launch = GK.bind_contract(d2, "abcd", a, "aebf", b, "dfce", force_gather=force_gather)
    launch(); launch()
    torch.cuda.synchronize(); GK.poll_status()
    assert torch.equal(d2, d)


def test_contraction_alpha_beta_and_three_index_case():
    """D_abc = alpha * sum_d A_bda B_dc + beta * C_abc (the contraction of the reference's benchmark,
    benchmarks/tensor-contractions/run.jl:10), scaled down."""
    rng = np.random.default_rng(31)
    ea, eb, ec, ed = 64, 32, 96, 128
    A = (rng.random((eb, ed, ea)) * 2 - 1).astype(np.float16)
    B = (rng.random((ed, ec)) * 2 - 1).astype(np.float16)
    Cm = rng.random((ea, eb, ec)).astype(np.float32)
    d = _julia_tensor(Cm)
    GK.contract_(d, "abc", _julia_tensor(A), "bda", _julia_tensor(B), "dc", alpha=2.0, beta=0.5)
    torch.cuda.synchronize(); GK.poll_status()
    want = O.contract(A, "bda", B, "dc", "abc", 2.0, 0.5, Cm)
    assert O.normwise_error(GK.to_numpy(d), want) <= TOL_TENSOR


@pytest.mark.parametrize("force_gather", [False, True])
def test_contraction_with_batch_modes(force_gather):
    """A label in A, B and D is a batch mode: D[m,n,p,q] = sum_k A[m,k,p,q] B[k,q,n,p] is one product per
    (p, q), each on its own slices (here 3 x 2 of them, B's batch strides permuted)."""
    rng = np.random.default_rng(21)
    m, n, k, p, q = 128, 96, 64, 3, 2
    A = rng.integers(-2, 3, (m, k, p, q)).astype(np.float16)
    B = rng.integers(-2, 3, (k, q, n, p)).astype(np.float16)
    Cm = rng.integers(-3, 4, (m, n, p, q)).astype(np.float32)
    d = _julia_tensor(Cm)
    GK.contract_(d, "mnpq", _julia_tensor(A), "mkpq", _julia_tensor(B), "kqnp", alpha=2.0, beta=1.0, force_gather=force_gather)
    torch.cuda.synchronize(); GK.poll_status()
    want = 2.0 * np.einsum("mkpq,kqnp->mnpq", A.astype(np.float32), B.astype(np.float32)) + Cm
    assert np.array_equal(GK.to_numpy(d), want)
    assert np.array_equal(want, O.contract(A, "mkpq", B, "kqnp", "mnpq", 2.0, 1.0, Cm))


def test_split_k_for_contractions_and_two_plane_products():
    """Few output tiles and a long contracted index: with a workspace the contraction (two-mode
    strides of D) and the complex product (two accumulator planes) are cut along K as well."""
    rng = np.random.default_rng(23)
    # D[a,b,c] = sum_{e,f} A[a,e,b,f] B[f,c,e]: M = (a,b) = 64*4, N = c = 128, K = (e,f) = 64*128 = 8192
    A = rng.integers(-2, 3, (64, 64, 4, 128)).astype(np.float16)
    B = rng.integers(-2, 3, (128, 128, 64)).astype(np.float16)
    a, b = _julia_tensor(A), _julia_tensor(B)
    d = GK.cuarray(GK.Float32, 64, 4, 128)
    plan = GK.contract_query(d, "abc", a, "aebf", b, "fce")
    assert plan.kernel == 1 and plan.workspace_bytes >= 2 * 256 * 128 * 4, (plan.kernel, plan.workspace_bytes)
    GK.contract_(d, "abc", a, "aebf", b, "fce")                  # the package lends the workspace
    torch.cuda.synchronize(); GK.poll_status()
    want = O.contract(A, "aebf", B, "fce", "abc")
    assert np.array_equal(GK.to_numpy(d), want)
    d2 = GK.cuarray(GK.Float32, 64, 4, 128)
    tiny = torch.zeros(64, dtype=torch.int64, device="cuda")       # too small to split: same numbers, unsplit
    GK.contract_(d2, "abc", a, "aebf", b, "fce", workspace=tiny)
    torch.cuda.synchronize(); GK.poll_status()
    assert torch.equal(d2, d)
    # planar complex, 256 x 256 x 8192, interleaved Complex{Float32} result with C and alpha/beta
    M, N, K = 256, 256, 8192
    Ac = rng.integers(-2, 3, (2, M, K)).astype(np.float16); Bc = rng.integers(-2, 3, (2, K, N)).astype(np.float16)
    Cc = rng.integers(-3, 4, (2, M, N)).astype(np.float32)
    dc = planar(Cc)
    conf = GK.get_config(gemm_shape=(M, N, K), operator=Operator.WMMAComplexOp[16, 16, 16, GK.Float16, GK.Float32],
                         global_a_layout=Layout.SplitColMajor[GK.Float16], global_b_layout=Layout.SplitColMajor[GK.Float16],
                         global_c_layout=Layout.SplitColMajor[GK.Float32], global_d_layout=Layout.SplitColMajor[GK.Float32],
                         block_shape=(64, 64, 32))
    pa, pb = planar(Ac), planar(Bc)
    assert GK.query(conf, pa, pb, dc, dc).workspace_bytes >= 2 * 2 * M * N * 4
    GK.matmul(conf, pa, pb, dc, dc, transform_shared_to_regs_a=Transform.Elementwise(Transform.Scale(2.0)))
    torch.cuda.synchronize(); GK.poll_status()
    re, im = O.complex_gemm(Ac[0], Ac[1], Bc[0], Bc[1], Cc[0], Cc[1], 2.0, 1.0)
    got = GK.to_numpy(dc)
    assert np.array_equal(got[..., 0], re) and np.array_equal(got[..., 1], im)


def test_contraction_errors():
    a = GK.cuarray(GK.Float16, 8, 8); b = GK.cuarray(GK.Float16, 8, 4); d = GK.cuarray(GK.Float32, 8, 8)
    with pytest.raises(GK.DimensionMismatch):
        GK.contract_(d, "ij", a, "ik", b, "kj")              # j: 8 vs 4
    with pytest.raises(Transform.UnsupportedFunctor):
        GK.contract_(d, "ij", a, "ij", GK.cuarray(GK.Float16, 8, 8), "ij")   # batched modes


# ------------------------------------------------------------------------------------------------
# Diagonal A (Layout.Diagonal): D = diag(v) * B + C
# ------------------------------------------------------------------------------------------------
def test_golden_diagonal(golden):
    cases, want = golden
    cs = cases["diagonal"]
    v, B, Cm = cs["A"], cs["B"], cs["C"]
    M, N = B.shape
    # as in the reference's harness: a full M x K matrix whose first column holds the diagonal
    Afull = np.zeros((M, M), dtype=np.float16); Afull[:, 0] = v
    c = dev(Cm); d = GK.cuarray(GK.Float32, M, N)
    conf = run_matmul(dev(Afull), dev(B), c, d, M=M, N=N, K=M, op=Operator.WMMAOp[16, 16, 16, GK.Float16, GK.Float32],
                      la=Layout.Diagonal[GK.Float16], lb=Layout.ColMajor[GK.Float16], lc=Layout.ColMajor[GK.Float32],
                      ld=Layout.ColMajor[GK.Float32], block_shape=(64, 64, 32),
                      shared_a_layout=Layout.Padded[Layout.UnsafeAlignedColMajor[GK.Float16], 8])
    assert GK.query(conf, dev(Afull), dev(B), c, d).kernel == 4
    assert O.normwise_error(GK.to_numpy(d), want["diagonal/D"]) <= 1e-6


@pytest.mark.parametrize("tb", [False, True])
def test_diagonal_4096_matches_oracle_and_dense_product(tb):
    """4096^2 (the size of the reference's diagonal benchmark): against the oracle, and against the
    dense tensor-core product with the same diagonal matrix written out in full."""
    n = 4096
    rng = np.random.default_rng(51 + tb)
    v = rng.random(n).astype(np.float16)
    B = rng.random((n, n)).astype(np.float16)
    Cm = rng.random((n, n)).astype(np.float32)
    b = dev(B.T.copy() if tb else B)
    lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[GK.Float16]
    c = dev(Cm); d = GK.cuarray(GK.Float32, n, n)
    run_matmul(dev(v), b, c, d, M=n, N=n, K=n, op=Operator.TCGen05Operator[GK.Float16, GK.Float32],
               la=Layout.Diagonal[GK.Float16], lb=lb, lc=Layout.UnsafeAlignedColMajor[GK.Float32],
               ld=Layout.UnsafeAlignedColMajor[GK.Float32], block_shape=(128, 128, 64),
               shared_a_layout=Layout.Padded[Layout.UnsafeAlignedColMajor[GK.Float16], 8])
    got = GK.to_numpy(d)
    assert O.normwise_error(got, O.diagonal_gemm(v, B, Cm)) <= 1e-6
    dense = GK.cuarray(GK.Float32, n, n); dense.copy_(c)
    GK.matmatmul_(dense, "N", "T" if tb else "N", dev(np.diag(v)), b, 1.0, 1.0)
    torch.cuda.synchronize()
    assert O.normwise_error(got, GK.to_numpy(dense)) <= 1e-6


# ------------------------------------------------------------------------------------------------
# replay of the reference's complex / dual configurations (configs/configs.jl:385-486, 656-695):
# interleaved Complex{Float16} global arrays, D = A*B + C
# ------------------------------------------------------------------------------------------------
def _interleaved(z_re, z_im, eltype):
    """two numpy planes (r, c) -> device array of (re, im) pairs, shape (2, r, c), strides (1, 2, 2r)"""
    return GK.to_cuarray(np.stack([z_re, z_im], axis=0), eltype)


@pytest.mark.parametrize("n", [128, 256, 2048])
@pytest.mark.parametrize("ta,tb,number", [(0, 0, "complex"), (0, 1, "complex"), (1, 0, "complex"), (1, 1, "complex"),
                                          (0, 0, "dual")])
def test_reference_complex_dual_configs_interleaved(n, ta, tb, number):
    rng = np.random.default_rng(n + 10 * ta + 100 * tb + (7 if number == "dual" else 0))
    A = rng.random((2, n, n)).astype(np.float16); B = rng.random((2, n, n)).astype(np.float16)
    Cm = rng.random((2, n, n)).astype(np.float32)
    a = _interleaved(A[0], A[1], GK.Float16); b = _interleaved(B[0], B[1], GK.Float16)
    c = _interleaved(Cm[0], Cm[1], GK.Float32); d = GK.cuarray(GK.ComplexF32, n, n)
    opcls = Operator.WMMAComplexOp if number == "complex" else Operator.WMMADualOp
    la = (Layout.InterleavedRowMajor if ta else Layout.InterleavedColMajor)[GK.Float16]
    lb = (Layout.InterleavedRowMajor if tb else Layout.InterleavedColMajor)[GK.Float16]
    conf = GK.get_config(
        gemm_shape=(n, n, n), operator=opcls[16, 16, 16, GK.Float16, GK.Float32],
        global_a_layout=la, global_b_layout=lb,
        global_c_layout=Layout.InterleavedColMajor[GK.Float32], global_d_layout=Layout.InterleavedColMajor[GK.Float32],
        shared_a_layout=Layout.Padded[(Layout.SplitRowMajor if ta else Layout.SplitColMajor)[GK.Float16], 8],
        shared_b_layout=Layout.Padded[(Layout.SplitRowMajor if tb else Layout.SplitColMajor)[GK.Float16], 8],
        shared_c_layout=Layout.SplitColMajor[GK.Float32], shared_d_layout=Layout.SplitColMajor[GK.Float32],
        warps_per_block=8, compute_warp=(16, 32, 16), block_shape=(64, 64, 32),
        mem_a_warp=(4, 32) if ta else (64, 2), mem_b_warp=(2, 64) if tb else (32, 4), mem_cd_warp=(64, 1),
        mem_a_thread=(1, 4) if ta else (4, 1), mem_b_thread=(1, 4) if tb else (4, 1), mem_cd_thread=(2, 1),
        is_a_col_major=not ta, is_b_col_major=not tb)
    plan = GK.query(conf, a, b, c, d)
    assert plan.kernel == 1 and plan.workspace_bytes == 2 * (2 * n * n * 2)
    GK.matmul(conf, a, b, c, d, kernel=Kernel.matmul_pipelined)
    torch.cuda.synchronize(); GK.poll_status()
    f = O.complex_gemm if number == "complex" else O.dual_gemm
    re, im = f(A[0], A[1], B[0], B[1], Cm[0], Cm[1], 1.0, 1.0, bool(ta), bool(tb))
    got = GK.to_numpy(d)                      # (2, n, n)
    assert O.normwise_error(got[0], re) <= TOL_TENSOR and O.normwise_error(got[1], im) <= TOL_TENSOR
    assert O.isapprox_elementwise(re, got[0], "Float16") or number == "complex"   # sums of positives only for dual/re


# ------------------------------------------------------------------------------------------------
# replay of the reference's configuration zoo (configs/configs.jl:492-653), one case per family,
# transpose pair and size class; alpha = 2, beta = 3 as there; elementwise sqrt(eps) rule
# ------------------------------------------------------------------------------------------------
FPU_TYPES = [("Float16", "Float32"), ("Float32", "Float32"), ("Float32", "Float64"), ("Float64", "Float64"),
             ("Int16", "Int16"), ("Int32", "Int32"), ("Int64", "Int64")]


@pytest.mark.parametrize("ab,cd", FPU_TYPES)
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("n", [128, 256])
def test_zoo_fpu_types(ab, cd, ta, tb, n):
    AB, CD = getattr(GK, ab), getattr(GK, cd)
    rng = np.random.default_rng(n + ta + 2 * tb)
    if AB.is_integer:
        info = np.iinfo(AB.np_dtype)
        A = rng.integers(info.min, info.max, (n, n), dtype=AB.np_dtype)
        B = rng.integers(info.min, info.max, (n, n), dtype=AB.np_dtype)
        Cm = rng.integers(info.min, info.max, (n, n), dtype=CD.np_dtype)
    else:
        A = rng.random((n, n)).astype(AB.np_dtype); B = rng.random((n, n)).astype(AB.np_dtype)
        Cm = rng.random((n, n)).astype(CD.np_dtype)
    c = dev(Cm); d = GK.cuarray(CD, n, n)
    la = (Layout.UnsafeAlignedRowMajor if ta else Layout.UnsafeAlignedColMajor)[AB]
    lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[AB]
    run_matmul(dev(A), dev(B), c, d, M=n, N=n, K=n, op=Operator.FPUOp[8, 16, 2, 4, 8, 1, AB, CD], la=la, lb=lb,
               lc=Layout.UnsafeAlignedColMajor[CD], ld=Layout.UnsafeAlignedColMajor[CD], alpha=2, beta=3,
               block_shape=(64, 64, 32))
    got = GK.to_numpy(d)
    if AB.is_integer:
        assert np.array_equal(got, O.integer_gemm(A, B, Cm, 2, 3, bool(ta), bool(tb)))
    else:
        want = O.gemm64(A, B, Cm, 2.0, 3.0, bool(ta), bool(tb))
        assert O.isapprox_elementwise(want, got, ab)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("mnk", [(128, 128, 128), (256, 256, 128), (128, 128, 256), (256, 256, 256)])
def test_zoo_tropical(ta, tb, mnk):
    M, N, K = mnk
    rng = np.random.default_rng(M + N + K + ta + 2 * tb)
    A = rng.random((K, M) if ta else (M, K)).astype(np.float32); B = rng.random((N, K) if tb else (K, N)).astype(np.float32)
    Cm = rng.random((M, N)).astype(np.float32)
    c = dev(Cm); d = GK.cuarray(GK.Float32, M, N)
    la = (Layout.UnsafeAlignedRowMajor if ta else Layout.UnsafeAlignedColMajor)[GK.Float32]
    lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[GK.Float32]
    run_matmul(dev(A), dev(B), c, d, M=M, N=N, K=K, op=Operator.TropicalFPUOp[8, 16, 2, 4, 8, 1, GK.Float32, GK.Float32],
               la=la, lb=lb, lc=Layout.UnsafeAlignedColMajor[GK.Float32], ld=Layout.UnsafeAlignedColMajor[GK.Float32],
               block_shape=(64, 64, 32))
    assert np.array_equal(GK.to_numpy(d), O.tropical_gemm(A, B, Cm, bool(ta), bool(tb)))


@pytest.mark.parametrize("cd,min_dim", [("Float16", 256), ("Float32", 128)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("op_shape", [(16, 16, 16), (8, 32, 16), (32, 8, 16)])
@pytest.mark.parametrize("zero_c", [False, True])
def test_zoo_wmma(cd, min_dim, ta, tb, op_shape, zero_c):
    """WMMA configurations (configs.jl:573-612): sizes {1,2} x min_dimension mixes and 2048^3,
    alpha = 2, beta = 3 (0 when C is Layout.Zero).  The WMMA operator shapes are accepted and run on
    the tcgen05 kernel."""
    CD = getattr(GK, cd)
    for (M, N, K) in [(min_dim, min_dim, min_dim), (2 * min_dim, 2 * min_dim, min_dim), (min_dim, min_dim, 2 * min_dim),
                      (2048, 2048, 2048)]:
        rng = np.random.default_rng(M + N + K)
        A = rng.random((K, M) if ta else (M, K)).astype(np.float16); B = rng.random((N, K) if tb else (K, N)).astype(np.float16)
        Cm = rng.random((M, N)).astype(CD.np_dtype)
        c = dev(Cm); d = GK.cuarray(CD, M, N)
        la = (Layout.UnsafeAlignedRowMajor if ta else Layout.UnsafeAlignedColMajor)[GK.Float16]
        lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[GK.Float16]
        beta = 0.0 if zero_c else 3.0
        run_matmul(dev(A), dev(B), None if zero_c else c, d, M=M, N=N, K=K,
                   op=Operator.WMMAOp[(*op_shape, GK.Float16, CD)], la=la, lb=lb,
                   lc=(Layout.Zero if zero_c else Layout.UnsafeAlignedColMajor)[CD], ld=Layout.UnsafeAlignedColMajor[CD],
                   alpha=2.0, beta=3.0, block_shape=(128, 128, 64), warps_per_block=8,
                   compute_warp=(32, 64, 16), kernel=Kernel.matmul_pipelined)
        want = O.gemm(A, B, Cm, 2.0, beta, bool(ta), bool(tb))
        assert O.isapprox_elementwise(want, GK.to_numpy(d), "Float16"), (M, N, K)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_zoo_wmma_parameter_sweep(ta, tb):
    """The parameter sweep of configs/configs.jl:597-612 at 256^3: block shapes with BLOCK_M * BLOCK_N <= 128^2,
    warp grids with at least four warps, zero_c, both kernels.  A combination the validity rules exclude
    raises ConfigError and counts as skipped (test/matmul.jl:22-24); every other one must run and match
    the oracle (alpha = 2, beta = 3, or 0 with Layout.Zero) under the reference's element-wise rule."""
    import itertools
    M = N = K = 256
    rng = np.random.default_rng(597 + 2 * ta + tb)
    A = rng.random((K, M) if ta else (M, K)).astype(np.float16); B = rng.random((N, K) if tb else (K, N)).astype(np.float16)
    Cm = rng.random((M, N)).astype(np.float32)
    a, b, c = dev(A), dev(B), dev(Cm)
    want = {False: O.gemm(A, B, Cm, 2.0, 3.0, bool(ta), bool(tb)), True: O.gemm(A, B, None, 2.0, 0.0, bool(ta), bool(tb))}
    la = (Layout.UnsafeAlignedRowMajor if ta else Layout.UnsafeAlignedColMajor)[GK.Float16]
    lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[GK.Float16]
    blocks = [blk for blk in itertools.product([64, 128, 256], [64, 128, 256], [16, 32, 64]) if blk[0] * blk[1] <= 128 * 128]
    grids = [w for w in itertools.product([1, 2, 4], [1, 2, 4]) if w[0] * w[1] >= 4]
    ran = skipped = 0
    for blk, (wm, wn), zero_c, kern in itertools.product(blocks, grids, [False, True],
                                                         [Kernel.matmul_singlestage, Kernel.matmul_pipelined]):
        d = GK.cuarray(GK.Float32, M, N)
        try:
            run_matmul(a, b, None if zero_c else c, d, M=M, N=N, K=K, op=Operator.WMMAOp[16, 16, 16, GK.Float16, GK.Float32],
                       la=la, lb=lb, lc=(Layout.Zero if zero_c else Layout.UnsafeAlignedColMajor)[GK.Float32],
                       ld=Layout.UnsafeAlignedColMajor[GK.Float32], alpha=2.0, beta=3.0, block_shape=blk,
                       warps_per_block=wm * wn, compute_warp=(blk[0] // wm, blk[1] // wn, 16), kernel=kern)
        except GK.ConfigError:
            skipped += 1
            continue
        ran += 1
        assert O.isapprox_elementwise(want[zero_c], GK.to_numpy(d), "Float16"), (blk, wm, wn, zero_c, kern)
    assert ran + skipped == 18 * 6 * 2 * 2
    assert ran >= 200 and skipped >= 50, (ran, skipped)       # the rules cut a good part of the sweep, and leave most of it


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("n", [128, 256, 4096])
def test_zoo_bias(ta, tb, n):
    """Bias configurations (configs.jl:615-633): per-column Float32 bias, alpha = beta = 1."""
    rng = np.random.default_rng(n + ta + 2 * tb)
    A = rng.random((n, n)).astype(np.float16); B = rng.random((n, n)).astype(np.float16)
    Cm = rng.random((n, n)).astype(np.float32); bias = rng.random((1, n)).astype(np.float32)
    c = dev(Cm); d = GK.cuarray(GK.Float32, n, n)
    la = (Layout.UnsafeAlignedRowMajor if ta else Layout.UnsafeAlignedColMajor)[GK.Float16]
    lb = (Layout.UnsafeAlignedRowMajor if tb else Layout.UnsafeAlignedColMajor)[GK.Float16]
    run_matmul(dev(A), dev(B), c, d, M=n, N=n, K=n, op=Operator.WMMAOp[16, 16, 16, GK.Float16, GK.Float32], la=la, lb=lb,
               lc=Layout.UnsafeAlignedColMajor[GK.Float32], ld=Layout.UnsafeAlignedColMajor[GK.Float32],
               epilogue=Epilogue.Bias(dev(bias.reshape(-1))), block_shape=(128, 128, 64), kernel=Kernel.matmul_pipelined)
    want = O.gemm(A, B, Cm, 1.0, 1.0, bool(ta), bool(tb)) + bias
    assert O.isapprox_elementwise(want, GK.to_numpy(d), "Float16")


# ------------------------------------------------------------------------------------------------
# randomised sweep over shapes, transposes, types, tile overrides and epilogues
# ------------------------------------------------------------------------------------------------
def _fuzz_cases(n=48):
    rng = np.random.default_rng(20240)
    cases = []
    for i in range(n):
        M, N, K = (int(rng.choice([8, 40, 136, 264, 520, 1032, 1544])) + 8 * int(rng.integers(0, 16)) for _ in range(3))
        cases.append(dict(i=i, M=M, N=N, K=K, ta=bool(rng.integers(2)), tb=bool(rng.integers(2)),
                          ab=str(rng.choice(["Float16", "BFloat16", "TF32"])), cd=str(rng.choice(["Float32", "same"])),
                          tile_n=int(rng.choice([0, 0, 64, 128, 256, 512])), cg=int(rng.choice([0, 1, 2])),
                          beta=float(rng.choice([0.0, 1.0, -0.5])), alpha=float(rng.choice([1.0, 2.0, 0.25])),
                          bias=str(rng.choice(["none", "row", "col"])), act=str(rng.choice(["none", "relu", "gelu"]))))
    return cases


@pytest.mark.parametrize("cs", _fuzz_cases(), ids=lambda c: f"{c['i']}-{c['M']}x{c['N']}x{c['K']}-{c['ab']}")
def test_randomised_shapes_types_tiles_and_epilogues(cs):
    rng = np.random.default_rng(1000 + cs["i"])
    M, N, K, ta, tb = cs["M"], cs["N"], cs["K"], cs["ta"], cs["tb"]
    tf32 = cs["ab"] == "TF32"
    AB = GK.Float32 if tf32 else getattr(GK, cs["ab"])
    CD = GK.Float32 if (cs["cd"] == "Float32" or tf32) else AB
    # multiples of 1/8 in [-1, 1]: exact in every input type, so the only rounding is the output's
    A = (rng.integers(-8, 9, (K, M) if ta else (M, K)) / 8).astype(np.float32)
    B = (rng.integers(-8, 9, (N, K) if tb else (K, N)) / 8).astype(np.float32)
    Cm = (rng.integers(-8, 9, (M, N)) / 8).astype(np.float32)
    bias = (rng.integers(-8, 9, M if cs["bias"] == "row" else N) / 8).astype(np.float32) if cs["bias"] != "none" else None
    if cs["tile_n"] == 512 and cs["cg"] == 1:
        cs = dict(cs, cg=2)
    kw = {}
    if cs["tile_n"]:
        kw["tile_n"] = cs["tile_n"]
    if cs["cg"]:
        kw["cta_group"] = cs["cg"]
    la = (Layout.RowMajor if ta else Layout.ColMajor)[AB]; lb = (Layout.RowMajor if tb else Layout.ColMajor)[AB]
    has_c = cs["beta"] != 0.0
    c = dev(Cm, CD) if has_c else None
    d = GK.cuarray(CD, M, N)
    opct = Operator.TF32 if tf32 else AB
    act = {"none": None, "relu": Transform.ReLU(), "gelu": Transform.GELU()}[cs["act"]]
    epi = Epilogue.Bias(torch.from_numpy(bias).cuda(), axis=cs["bias"]) if bias is not None else None
    try:
        run_matmul(dev(A, AB), dev(B, AB), c, d, M=M, N=N, K=K, op=Operator.TCGen05Operator[opct, GK.Float32], la=la, lb=lb,
                   lc=(Layout.ColMajor if has_c else Layout.Zero)[CD], ld=Layout.ColMajor[CD],
                   alpha=cs["alpha"], beta=cs["beta"] if has_c else 1.0, epilogue=epi, act=act, **kw)
    except GK.ConfigError as e:
        pytest.skip(f"engine refuses this combination, as the reference's tests allow: {e}")
    want = cs["alpha"] * (( A.T if ta else A).astype(np.float64) @ (B.T if tb else B).astype(np.float64))
    if has_c:
        want = want + cs["beta"] * GK.to_numpy(c).astype(np.float64)
    want = O.epilogue(want, bias, cs["bias"] if bias is not None else "col", None if cs["act"] == "none" else cs["act"])
    tol = {"Float32": 2e-6, "Float16": 1e-3, "BFloat16": 8e-3}[CD.name]
    assert O.normwise_error(GK.to_numpy(d).astype(np.float64), want) <= tol


# ------------------------------------------------------------------------------------------------
# randomised contractions: mode orders, extents, both paths
# ------------------------------------------------------------------------------------------------
def _contraction_cases(n=24):
    rng = np.random.default_rng(777)
    cases = []
    for i in range(n):
        n_m, n_n, n_k = (int(rng.integers(1, 3)) for _ in range(3))        # 1-2 modes per group
        names = iter("abcdefgh")
        m_modes = [next(names) for _ in range(n_m)]; n_modes = [next(names) for _ in range(n_n)]
        k_modes = [next(names) for _ in range(n_k)]
        ext = {ch: int(rng.choice([8, 16, 32, 64])) for ch in m_modes + n_modes + k_modes}
        perm = lambda xs: "".join(rng.permutation(xs))
        cases.append(dict(i=i, a=perm(m_modes + k_modes), b=perm(k_modes + n_modes), d=perm(m_modes + n_modes), ext=ext,
                          alpha=float(rng.choice([1.0, 0.5])), beta=float(rng.choice([0.0, 1.0])),
                          force_gather=bool(rng.integers(0, 4) == 0)))
    return cases


@pytest.mark.parametrize("cs", _contraction_cases(), ids=lambda c: f"{c['i']}-{c['d']}={c['a']}*{c['b']}")
def test_randomised_contractions(cs):
    rng = np.random.default_rng(5000 + cs["i"])
    shape = lambda modes: tuple(cs["ext"][ch] for ch in modes)
    A = rng.integers(-2, 3, shape(cs["a"])).astype(np.float16)
    B = rng.integers(-2, 3, shape(cs["b"])).astype(np.float16)
    Cm = rng.integers(-4, 5, shape(cs["d"])).astype(np.float32)
    d = _julia_tensor(Cm)
    plan = GK.contract_query(d, cs["d"], _julia_tensor(A), cs["a"], _julia_tensor(B), cs["b"], cs["alpha"], cs["beta"],
                             force_gather=cs["force_gather"])
    assert plan.kernel in (1, 5) and (plan.kernel == 5 or not cs["force_gather"])
    GK.contract_(d, cs["d"], _julia_tensor(A), cs["a"], _julia_tensor(B), cs["b"], cs["alpha"], cs["beta"],
                 force_gather=cs["force_gather"])
    torch.cuda.synchronize(); GK.poll_status()
    want = O.contract(A, cs["a"], B, cs["b"], cs["d"], cs["alpha"], cs["beta"], Cm)
    assert np.array_equal(GK.to_numpy(d), want.astype(np.float32))        # small integers, alpha a power of two: exact
