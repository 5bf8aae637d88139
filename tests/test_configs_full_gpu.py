"""The benchmark configurations at their stated sizes: the CUDA path through the C ABI against the CPU
oracle on the same seeded inputs.  A full CPU product of these sizes takes minutes, so each result is
checked on sampled rows (every element of a row needs the whole of B and all of K, so a sampled row
exercises every k-block and every column tile), plus a checksum property over the whole result.

Tolerances (normwise relative error): <= 1e-5 for the FP32 FPU operator against a float64 product,
<= 1e-3 for the FP16/BF16 tensor-core paths.
"""
import numpy as np
import pytest
import torch

import gemmkernels_b200 as GK
from gemmkernels_b200 import Epilogue, Layout, Operator, Transform
from oracle import gemm_oracle as O

pytestmark = pytest.mark.gpu


def _dev(x, eltype=None):
    return GK.to_cuarray(np.asarray(x), eltype)


def _planar(x):
    t = torch.from_numpy(np.ascontiguousarray(np.asarray(x).transpose(0, 2, 1)))   # [2, c, r]
    return t.cuda().permute(2, 1, 0)


def test_config2_fp32_fpu_4096_transposed_a_bias_relu():
    """Configuration 2: D = ReLU(A*B + bias), FP32 ~ N(0,1), 4096^3, A stored transposed (K x M),
    bias of length M, FPUOp (no tensor cores).  64 sampled rows against the float64 product."""
    n = 4096
    At, B, bias = O.inputs_fp32_bias_relu(2, n, n, n)
    a, b, bias_d = _dev(At), _dev(B), _dev(bias)
    d = GK.cuarray(GK.Float32, n, n)
    conf = GK.get_config(gemm_shape=(n, n, n), operator=Operator.FPUOp[8, 8, 1, 4, 8, 1, GK.Float32, GK.Float32],
                         global_a_layout=Layout.UnsafeAlignedRowMajor[GK.Float32],
                         global_b_layout=Layout.UnsafeAlignedColMajor[GK.Float32],
                         global_c_layout=Layout.Zero[GK.Float32],
                         global_d_layout=Layout.UnsafeAlignedColMajor[GK.Float32],
                         is_a_col_major=False, is_b_col_major=True)
    epi = Epilogue.Bias(bias_d, axis="row")
    relu = Transform.Elementwise(Transform.ReLU())
    plan = GK.query(conf, a, b, None, d, epilogue=epi, transform_shared_to_global_d=relu)
    assert plan.kernel == 2, "configuration 2 must run on the FP32 FFMA kernel"
    GK.matmul(conf, a, b, None, d, epilogue=epi, transform_shared_to_global_d=relu)
    torch.cuda.synchronize(); GK.poll_status()
    rows = np.sort(np.random.default_rng(2).choice(n, 64, replace=False))
    acc = At[:, rows].astype(np.float64).T @ B.astype(np.float64) + bias[rows, None].astype(np.float64)
    want = np.maximum(acc, 0.0)
    got = d[torch.from_numpy(rows).cuda()].cpu().numpy()
    assert O.normwise_error(got, want) <= 1e-5
    assert (got >= 0).all()
    # ReLU zeroes exactly the entries whose pre-activation is negative (away from rounding distance)
    clear = np.abs(acc) > 1e-3
    assert np.array_equal((got > 0)[clear], (acc > 0)[clear])


def test_config3_dual_numbers_4096_sampled():
    """Configuration 3, dual-number variant: planar FP16 ~ U[-1,1), 4096^3, value and derivative
    planes accumulated in FP32 (three real products)."""
    n = 4096
    A, B = O.inputs_planar_fp16(3, n, n, n)
    a, b = _planar(A), _planar(B)
    d = GK.cuarray(GK.Float32, n, n, 2)
    conf = GK.get_config(gemm_shape=(n, n, n), operator=Operator.WMMADualOp[16, 16, 16, GK.Float16, GK.Float32],
                         global_a_layout=Layout.SplitColMajor[GK.Float16], global_b_layout=Layout.SplitColMajor[GK.Float16],
                         global_c_layout=Layout.Zero[GK.Float32], global_d_layout=Layout.SplitColMajor[GK.Float32],
                         block_shape=(64, 64, 32))
    assert GK.query(conf, a, b, None, d).kernel == 1
    GK.matmul(conf, a, b, None, d)
    torch.cuda.synchronize(); GK.poll_status()
    rows = np.sort(np.random.default_rng(3).choice(n, 64, replace=False))
    val, der = O.dual_gemm(A[0][rows], A[1][rows], B[0], B[1])
    got = d[torch.from_numpy(rows).cuda()].cpu().numpy()      # (64, n, 2)
    assert O.normwise_error(got[..., 0], val) <= 1e-3
    assert O.normwise_error(got[..., 1], der) <= 1e-3
    # the value plane of a dual product is the plain real product of the value planes
    d_real = GK.cuarray(GK.Float32, n, n)
    GK.mul_(d_real, a[..., 0], b[..., 0])
    torch.cuda.synchronize()
    assert torch.equal(d[..., 0], d_real)


def test_config5_bf16_16384_single_gpu_sampled():
    """Configuration 5 on one GPU: BF16 ~ N(0, 0.02), 16384^3, FP32 result.  64 sampled rows against
    the oracle, and a column-sum checksum of the whole result: 1'(A B) = (1'A) B."""
    n = 16384
    A, B = O.inputs_bf16_normal(5, n, n, n)
    a, b = _dev(A, GK.BFloat16), _dev(B, GK.BFloat16)
    d = GK.cuarray(GK.Float32, n, n)
    conf = GK.get_config(gemm_shape=(n, n, n), operator=Operator.TCGen05Operator[GK.BFloat16, GK.Float32],
                         global_a_layout=Layout.UnsafeAlignedColMajor[GK.BFloat16],
                         global_c_layout=Layout.Zero[GK.Float32],
                         global_d_layout=Layout.UnsafeAlignedColMajor[GK.Float32])
    assert GK.query(conf, a, b, None, d).kernel == 1
    GK.matmul(conf, a, b, None, d)
    torch.cuda.synchronize(); GK.poll_status()
    rows = np.sort(np.random.default_rng(5).choice(n, 64, replace=False))
    want = O.gemm(A[rows], B)
    got = d[torch.from_numpy(rows).cuda()].cpu().numpy()
    assert O.normwise_error(got, want) <= 1e-3
    ones_a = A.sum(axis=0, dtype=np.float64)                  # 1'A, length K
    want_sum = np.concatenate([ones_a @ B[:, j:j + 2048].astype(np.float64) for j in range(0, n, 2048)])
    got_sum = d.double().sum(dim=0).cpu().numpy()
    assert O.normwise_error(got_sum, want_sum) <= 1e-3
