"""The column-sharded GEMM behind the C ABI (gk_mgpu_*): one rank per GPU, NCCL found by the library.

The single-GPU test joins a communicator of one rank (dlopen of NCCL, init, the fall-through to the
plain paths, destroy).  The two-rank test needs two GPUs and runs one process per GPU: the device form
with A broadcast in K-panels under the product, and the host form (every rank uploads half of A, NCCL
all-gathers assemble it chunk by chunk), both against the oracle on small-integer inputs (exact)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _host_colmajor(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x.T)).to(dtype).pin_memory().T


def _conf(GK, M, N, K, trans_a=False, with_c=False):
    from gemmkernels_b200 import Layout, Operator
    la = (Layout.RowMajor if trans_a else Layout.ColMajor)[GK.Float16]
    return GK.get_config(gemm_shape=(M, N, K), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                         global_a_layout=la, global_b_layout=Layout.ColMajor[GK.Float16],
                         global_c_layout=(Layout.ColMajor if with_c else Layout.Zero)[GK.Float32],
                         global_d_layout=Layout.ColMajor[GK.Float32], is_a_col_major=not trans_a)


def test_communicator_of_one_rank_falls_through_to_the_plain_paths():
    import gemmkernels_b200 as GK
    from gemmkernels_b200 import multigpu
    from oracle import gemm_oracle as O
    assert multigpu.init() == (0, 1)
    try:
        rng = np.random.default_rng(3)
        M, N, K = 512, 384, 2048
        A = rng.integers(-2, 3, (M, K)).astype(np.float32); B = rng.integers(-2, 3, (K, N)).astype(np.float32)
        conf = _conf(GK, M, N, K)
        a, b, d = GK.to_cuarray(A, GK.Float16), GK.to_cuarray(B, GK.Float16), GK.cuarray(GK.Float32, M, N)
        multigpu.colshard_matmul_device(conf, a, b, None, d, a_mode="broadcast", root=0)
        multigpu.broadcast_a_library(a)
        torch.cuda.synchronize(); GK.poll_status()
        assert np.array_equal(GK.to_numpy(d), O.gemm(A, B))
        dh = torch.empty(N, M, dtype=torch.float32).pin_memory().T
        multigpu.colshard_matmul_host(conf, _host_colmajor(A, torch.float16), _host_colmajor(B, torch.float16), None, dh)
        assert np.array_equal(dh.numpy(), O.gemm(A, B))
    finally:
        multigpu.shutdown()


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import gemmkernels_b200 as GK
    from gemmkernels_b200 import Epilogue, Transform, multigpu
    from oracle import gemm_oracle as O
    try:
        assert multigpu.init(device_index=rank) == (rank, world)
        rng = np.random.default_rng(17)                         # the same A on every rank
        # --- device operands, A broadcast from rank 1 in K-panels under the product
        M, K, n_total = 1024, 4096, 1280
        A = rng.integers(-2, 3, (M, K)).astype(np.float32)
        B = rng.integers(-2, 3, (K, n_total)).astype(np.float32)
        Cm = rng.integers(-4, 5, (M, n_total)).astype(np.float32)
        bias = rng.integers(-3, 4, M).astype(np.float32)
        shard = multigpu.column_shard(n_total, world, rank, 256)
        cols = slice(shard.start, shard.stop)
        conf = _conf(GK, M, shard.count, K, with_c=True)
        a = GK.to_cuarray(A if rank == 1 else np.zeros_like(A), GK.Float16)
        b, c = GK.to_cuarray(B[:, cols], GK.Float16), GK.to_cuarray(Cm[:, cols])
        d = GK.cuarray(GK.Float32, M, shard.count)
        epi = Epilogue.Bias(torch.from_numpy(bias).cuda(), axis="row")
        relu = Transform.Elementwise(Transform.ReLU())
        for panels in (0, 1, 4):
            if rank != 1:
                a.zero_()
            multigpu.colshard_matmul_device(conf, a, b, c, d, a_mode="broadcast", root=1, k_panels=panels, epilogue=epi,
                                            transform_shared_to_global_d=relu)
            torch.cuda.synchronize(); GK.poll_status()
            want = np.maximum(A @ B[:, cols] + Cm[:, cols] + bias[:, None], 0)
            assert np.array_equal(GK.to_numpy(d), want), ("device", panels)
            assert np.array_equal(GK.to_numpy(a), A), "A must have arrived on every rank"
        # a transposed A (stored K x M) travels in panels of M: independent row blocks of D
        conf_t = _conf(GK, M, shard.count, K, trans_a=True, with_c=True)
        at = GK.to_cuarray(A.T.copy() if rank == 1 else np.zeros((K, M), np.float32), GK.Float16)
        for panels in (0, 2, 3):
            if rank != 1:
                at.zero_()
            d.zero_()
            multigpu.colshard_matmul_device(conf_t, at, b, c, d, a_mode="broadcast", root=1, k_panels=panels, epilogue=epi,
                                            transform_shared_to_global_d=relu)
            torch.cuda.synchronize(); GK.poll_status()
            assert np.array_equal(GK.to_numpy(d), want), ("device, transposed A", panels)
            assert np.array_equal(GK.to_numpy(at), A.T)
        # resident form: nothing is exchanged
        multigpu.colshard_matmul_device(conf, a, b, c, d, a_mode="resident", epilogue=epi, transform_shared_to_global_d=relu)
        torch.cuda.synchronize()
        assert np.array_equal(GK.to_numpy(d), want)
        # --- host operands: each rank uploads its share of every chunk of A; all-gathers assemble it
        for trans_a in (False, True):
            M, K = 4096, 8192                                   # 64 MiB of Float16: two chunks
            A = rng.integers(-2, 3, (M, K)).astype(np.float32)
            B = rng.integers(-2, 3, (K, n_total)).astype(np.float32)
            Cm = rng.integers(-4, 5, (M, n_total)).astype(np.float32)
            bias = rng.integers(-3, 4, M).astype(np.float32)
            conf = _conf(GK, M, shard.count, K, trans_a=trans_a, with_c=True)
            assert multigpu.host_plan(conf, world)[0] == 2
            ah = _host_colmajor(A.T if trans_a else A, torch.float16)
            bh, ch = _host_colmajor(B[:, cols], torch.float16), _host_colmajor(Cm[:, cols], torch.float32)
            dh = torch.empty(shard.count, M, dtype=torch.float32).pin_memory().T
            want = np.maximum(A @ B[:, cols] + Cm[:, cols] + bias[:, None], 0)
            for _ in range(2):                                  # the second call reuses buffers, streams and events
                dh.zero_()
                t = multigpu.colshard_matmul_host(conf, ah, bh, ch, dh, epilogue=Epilogue.Bias(torch.from_numpy(bias), axis="row"),
                                                  transform_shared_to_global_d=relu, device_index=rank, times=True)
                assert np.array_equal(dh.numpy(), want), ("host", trans_a)
            assert t["chunks"] == 2 and t["h2d_bytes"] == M * K * 2 // world + K * shard.count * 2 + M * shard.count * 4 + M * 4
            assert t["d2h_bytes"] == M * shard.count * 4 and t["total_ms"] > 0
        with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
            f.write("ok")
    finally:
        multigpu.shutdown(rank)
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_colshard_device_and_host(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.ok").exists()
