"""gk_gemm_host / matmul_host: operands and result in host memory.  Small problems take the plain
copy-compute-copy path; large real products are cut into blocks whose transfers and kernels overlap."""
import numpy as np
import pytest
import torch

import gemmkernels_b200 as GK
from gemmkernels_b200 import Epilogue, Layout, Operator, Transform
from oracle import gemm_oracle as O

pytestmark = pytest.mark.gpu


def host_colmajor(x: np.ndarray, dtype):
    """numpy (r, c) -> pinned CPU tensor of shape (r, c) with column-major strides."""
    return torch.from_numpy(np.ascontiguousarray(x.T)).to(dtype).pin_memory().T


@pytest.mark.parametrize("M,N,K,ta,tb,with_c", [
    (300, 200, 136, False, False, True),        # small: plain path
    (5120, 4608, 8192, False, False, True),     # 3 row chunks x 2 column chunks, C and a row bias
    (4096, 6000, 8192, True, True, False),      # both operands transposed, ragged last column chunk
])
def test_matmul_host_matches_oracle(M, N, K, ta, tb, with_c):
    rng = np.random.default_rng(M + N + K)
    A = rng.integers(-2, 3, (K, M) if ta else (M, K)).astype(np.float32)
    B = rng.integers(-2, 3, (N, K) if tb else (K, N)).astype(np.float32)
    Cm = rng.integers(-8, 9, (M, N)).astype(np.float32) if with_c else None
    bias = rng.integers(-4, 5, M).astype(np.float32) if with_c else None
    a, b = host_colmajor(A, torch.float16), host_colmajor(B, torch.float16)
    c = host_colmajor(Cm, torch.float32) if with_c else None
    d = torch.empty(N, M, dtype=torch.float32).pin_memory().T
    la = (Layout.RowMajor if ta else Layout.ColMajor)[GK.Float16]
    lb = (Layout.RowMajor if tb else Layout.ColMajor)[GK.Float16]
    conf = GK.get_config(gemm_shape=(M, N, K), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                         global_a_layout=la, global_b_layout=lb,
                         global_c_layout=(Layout.ColMajor if with_c else Layout.Zero)[GK.Float32],
                         global_d_layout=Layout.ColMajor[GK.Float32], is_a_col_major=not ta, is_b_col_major=not tb)
    kw = dict(epilogue=Epilogue.Bias(torch.from_numpy(bias), axis="row"),
              transform_shared_to_global_d=Transform.Elementwise(Transform.ReLU())) if with_c else {}
    for _ in range(2):                               # second call reuses streams, events and staging buffers
        d.zero_()
        GK.matmul_host(conf, a, b, c, d, **kw)
    rows = np.sort(rng.choice(M, min(M, 48), replace=False))
    Aop = (A.T if ta else A)[rows]
    want = Aop @ (B.T if tb else B)                  # small integers: exact in float32
    if with_c:
        want = np.maximum(want + Cm[rows] + bias[rows, None], 0)
    assert np.array_equal(d.numpy()[rows], want)
    # the rest of D is covered through a checksum against the device-resident product
    dd = GK.cuarray(GK.Float32, M, N)
    GK.matmul(conf, GK.to_cuarray(A, GK.Float16), GK.to_cuarray(B, GK.Float16),
              GK.to_cuarray(Cm) if with_c else None, dd,
              **({"epilogue": Epilogue.Bias(torch.from_numpy(bias).cuda(), axis="row"),
                  "transform_shared_to_global_d": Transform.Elementwise(Transform.ReLU())} if with_c else {}))
    torch.cuda.synchronize(); GK.poll_status()
    assert torch.equal(dd.cpu(), d)


def test_matmul_host_with_a_resident_on_the_device():
    """a_on_device: A is a device array used in place (the sharded path after a broadcast); B, D in host memory.
    Large enough for the column-chunk pipeline (D alone is 128 MiB)."""
    M, N, K = 4096, 8192, 2048
    rng = np.random.default_rng(99)
    A = rng.integers(-2, 3, (M, K)).astype(np.float32); B = rng.integers(-2, 3, (K, N)).astype(np.float32)
    a_dev = GK.to_cuarray(A, GK.Float16)
    b = host_colmajor(B, torch.float16)
    d = torch.zeros(N, M, dtype=torch.float32).pin_memory().T
    conf = GK.get_config(gemm_shape=(M, N, K), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                         global_a_layout=Layout.ColMajor[GK.Float16], global_c_layout=Layout.Zero[GK.Float32],
                         global_d_layout=Layout.ColMajor[GK.Float32])
    for _ in range(2):
        d.zero_()
        GK.matmul_host(conf, a_dev, b, None, d, a_on_device=True)
    rows = np.sort(rng.choice(M, 32, replace=False))
    assert np.array_equal(d.numpy()[rows], A[rows] @ B)
    assert float(d.abs().sum()) == float(np.abs(A @ B).sum())
