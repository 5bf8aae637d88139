"""Host logic of the column-block sharding (the N > 1 path of bench.py), exercised with two CPU ranks
over gloo.  The per-rank GEMM itself is a CUDA kernel and is not run here: a float32 product from
the oracle stands in for it, which is enough to check partitioning, the broadcast of A and the
assembly of D."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gemmkernels_b200 import multigpu


@pytest.mark.parametrize("n,world,multiple", [(16384, 8, 256), (8192, 2, 256), (1000, 4, 128), (5, 8, 1), (0, 3, 64),
                                              (16384, 3, 256)])
def test_column_shards_cover_the_columns_exactly(n, world, multiple):
    shards = [multigpu.column_shard(n, world, r, multiple) for r in range(world)]
    assert shards[0].start == 0 and shards[-1].stop == n
    for a, b in zip(shards, shards[1:]):
        assert a.stop == b.start
    assert sum(s.count for s in shards) == n
    assert all(s.count >= 0 for s in shards)
    # balanced to within one tile, and whole tiles except at the very end
    full = [s for s in shards if s.stop < n]
    assert all(s.count % multiple == 0 for s in full)
    assert max(s.count for s in shards) - min(s.count for s in shards) <= multiple


def test_column_shard_rejects_bad_ranks():
    with pytest.raises(ValueError):
        multigpu.column_shard(10, 2, 2)
    with pytest.raises(ValueError):
        multigpu.column_shard(10, 0, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, k, m, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import gemm_oracle as O
        rng = np.random.default_rng(123)
        A = rng.standard_normal((m, k)).astype(np.float32)
        B = rng.standard_normal((k, n)).astype(np.float32)
        shard = multigpu.column_shard(n, world, rank, 4)
        # column-major storage: A as (k, m) contiguous, blocks of B / D as (cols, k) / (cols, m)
        a_store = torch.from_numpy(np.ascontiguousarray(A.T)) if rank == 0 else torch.zeros(k, m)
        b_block = torch.from_numpy(np.ascontiguousarray(B[:, shard.start:shard.stop].T))
        d_block = torch.zeros(shard.count, m)

        def local_product(a_s, b_s, d_s):      # stand-in for the CUDA GEMM of one rank
            d_s.copy_(torch.from_numpy(np.ascontiguousarray(O.gemm(a_s.numpy().T, b_s.numpy().T).T)))

        multigpu.colshard_matmul(local_product, a_store, b_block, d_block)
        assert torch.equal(a_store, torch.from_numpy(np.ascontiguousarray(A.T)))       # A arrived everywhere
        # second step with A resident: no broadcast, new B block
        multigpu.colshard_matmul(local_product, a_store, b_block * 2, d_block, a_is_resident=True)
        # the host-path scheme: every rank contributes 1/world of each row chunk of A and an all-gather
        # assembles the chunk everywhere (gloo here, NCCL inside the library on GPUs)
        for trans_a in (False, True):
            chunks, rows = 3, 4
            got = multigpu.allgather_a_chunks(torch.from_numpy(A), trans_a, rank, world, chunks, rows)
            assert len(got) == chunks
            for i, chunk in enumerate(got):
                assert np.array_equal(chunk.numpy(), A[i * rows:(i + 1) * rows]), (trans_a, i)
        full = multigpu.gather_columns(d_block, shard)
        want = 2 * (A @ B)
        err = np.linalg.norm(full.numpy().T - want) / np.linalg.norm(want)
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(f"{err:.3e} {tuple(full.shape)}")
        assert err < 1e-5 and tuple(full.shape) == (n, m)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_colshard(tmp_path):
    world, n, k, m = 2, 22, 16, 12         # 22 columns in units of 4: blocks of 12 and 10
    mp.spawn(_worker, args=(world, _free_port(), n, k, m, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err, shape = (tmp_path / f"rank{r}.txt").read_text().split(" ", 1)
        assert float(err) < 1e-5 and shape == "(22, 12)"


def test_host_plan_of_the_sharded_host_path():
    """gk_mgpu_host_plan: chunk arithmetic of the library, no GPU needed."""
    import gemmkernels_b200 as GK
    from gemmkernels_b200 import Layout, Operator
    def conf(m, n, k, trans_a=False):
        la = (Layout.RowMajor if trans_a else Layout.ColMajor)[GK.Float16]
        return GK.get_config(gemm_shape=(m, n, k), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                             global_a_layout=la, global_c_layout=Layout.Zero[GK.Float32],
                             global_d_layout=Layout.ColMajor[GK.Float32], is_a_col_major=not trans_a)
    # 8192 x 8192 Float16 = 128 MiB -> four chunks of 2048 rows
    assert multigpu.host_plan(conf(8192, 1024, 8192), 8) == (4, 2048)
    # 16384^2 BFloat16-sized A (512 MiB) -> the cap of eight chunks
    assert multigpu.host_plan(conf(16384, 2048, 16384), 8) == (8, 2048)
    # small A: one chunk of all rows
    assert multigpu.host_plan(conf(1000, 64, 512), 2) == (1, 1000)
    # chunks of a transposed A are dealt out by rows: whole multiples of lcm(256, world)
    chunks, rows = multigpu.host_plan(conf(12288, 512, 8192, trans_a=True), 3)
    assert rows % 768 == 0 and chunks * rows >= 12288
    with pytest.raises(GK.ConfigError):
        multigpu.host_plan(conf(4096, 64, 1000), 3)          # K not divisible by the ranks
