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
        # the host-path variant: only rank 0 holds A in host memory; the per-rank host GEMM is replaced by
        # the same stand-in (there is no CUDA here), which must find A in place and be told so
        import importlib
        mm = importlib.import_module("gemmkernels_b200.matmul")     # the package re-exports a function of that name
        seen = {}

        def fake_matmul_host(conf, a, b, c, d, *, device_index=None, a_on_device=False, **kw):
            seen["a_on_device"] = a_on_device
            local_product(a.T, b.T, d.T)
        real, mm.matmul_host = mm.matmul_host, fake_matmul_host
        try:
            a_dev = torch.zeros(k, m).T                        # column-major (m, k) "device" array
            d_host = torch.zeros(shard.count, m).T
            multigpu.colshard_matmul_host(None, torch.from_numpy(np.ascontiguousarray(A.T)).T if rank == 0 else None,
                                          a_dev, (b_block * 2).T, d_host)
        finally:
            mm.matmul_host = real
        assert seen["a_on_device"] is True and torch.equal(a_dev.T, torch.from_numpy(np.ascontiguousarray(A.T)))
        assert torch.equal(d_host.T, d_block)
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
