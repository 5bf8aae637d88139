"""Column-block sharding of one large GEMM over the GPUs of a box (one process per GPU).

    D[:, J_r] = A * B[:, J_r]        rank r owns the column block J_r of B and of D

The blocks are independent; the only exchange is A.  Two layers:
  * `init` / `colshard_matmul_device` / `colshard_matmul_host` drive the library's own entry points
    (gk_mgpu_*): NCCL inside the C library, A broadcast in K-panels that overlap the product, or —
    from host memory — uploaded in shares over every rank's PCIe link and all-gathered over NVLink;
  * `column_shard`, `broadcast_a`, `colshard_matmul`, `gather_columns` are the partition arithmetic and
    a `torch.distributed` form of the same scheme (what the CPU tests run over gloo).
Kernels read local memory only: no peer loads, no multicast.  The reference has no multi-GPU path;
this is the partitioning named for the 16384^3 BFloat16 configuration.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ColumnShard:
    rank: int
    world: int
    n_total: int
    start: int       # first column of this rank's block
    count: int       # columns in the block

    @property
    def stop(self) -> int:
        return self.start + self.count


def column_shard(n_total: int, world: int, rank: int, multiple: int = 1) -> ColumnShard:
    """Contiguous column block of `rank`: blocks differ by at most `multiple` columns, every block
    but possibly the last is a multiple of `multiple` (use the tile width so no rank gets a ragged
    tile it could have avoided), blocks cover [0, n_total) exactly, empty blocks are allowed."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if n_total < 0 or multiple < 1:
        raise ValueError("n_total must be >= 0 and multiple >= 1")
    units = -(-n_total // multiple)                 # ceil
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    start, stop = min(u0 * multiple, n_total), min(u1 * multiple, n_total)
    return ColumnShard(rank, world, n_total, start, stop - start)


def broadcast_a(a_storage, src: int = 0, group=None):
    """Sends A from `src` to every rank, in place.  `a_storage` must be the contiguous storage of A
    (for a column-major device array `a` that is `a.T`).  Returns the tensor."""
    import torch.distributed as dist
    if not a_storage.is_contiguous():
        raise ValueError("broadcast_a needs the contiguous storage view of A (a.T for a column-major array)")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(a_storage, src=src, group=group)
    return a_storage


def colshard_matmul(local_product, a_storage, b_block, d_block, *, src: int = 0, group=None, a_is_resident=False):
    """One sharded product on this rank: broadcast A (unless it is already resident from an earlier
    call) and run `local_product(a_storage, b_block, d_block)` on the rank's own column block.
    `local_product` is the single-GPU GEMM (e.g. a closure over `GemmKernels.matmul`)."""
    if not a_is_resident:
        broadcast_a(a_storage, src, group)
    local_product(a_storage, b_block, d_block)
    return d_block


# ------------------------------------------------------------------------------------------------
# the sharded path behind the C ABI (gk_mgpu_*): one rank per GPU, NCCL found by the library itself
# ------------------------------------------------------------------------------------------------
_joined: dict = {}


def init(group=None, device_index=None):
    """Joins this rank's handle to the library's communicator (collective).  The 128-byte NCCL id is
    made on rank 0 and handed round with `torch.distributed` (any transport would do: the C entry
    points only need the bytes).  Idempotent per device."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from . import _lib as L
    from .matmul import _raise, handle
    dev = device_index if device_index is not None else torch.cuda.current_device()
    if dev in _joined:
        return _joined[dev]
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    ident = C.create_string_buffer(L.GK_MGPU_UNIQUE_ID_BYTES)
    if rank == 0:
        st = L.lib.gk_mgpu_unique_id(ident)
        if st != L.GK_OK:
            _raise(st)
    box = [bytes(ident.raw)]
    if world > 1:
        dist.broadcast_object_list(box, src=0, group=group)
    with torch.cuda.device(dev):
        st = L.lib.gk_mgpu_init(handle(dev), rank, world, C.c_char_p(box[0]))
    if st != L.GK_OK:
        _raise(st)
    _joined[dev] = (rank, world)
    return rank, world


def shutdown(device_index=None):
    """Leaves the communicator (collective); the handle itself stays usable."""
    import torch
    from . import _lib as L
    from .matmul import handle
    dev = device_index if device_index is not None else torch.cuda.current_device()
    if _joined.pop(dev, None) is not None:
        L.lib.gk_mgpu_destroy(handle(dev))


def host_plan(conf, world: int):
    """(chunks, rows per chunk) `colshard_matmul_host` cuts A into for this configuration; host
    arithmetic of the library (gk_mgpu_host_plan), needs no GPU."""
    import ctypes as C
    from . import _lib as L
    from .matmul import _raise
    M, N, K = (conf.matmul_shape[k] for k in "MNK")
    et = conf.global_a_layout.eltype
    desc = L.GemmDesc(m=M, n=N, k=K, trans_a=0 if conf.global_a_layout.col_major else 1, dtype_a=et.gk, dtype_b=et.gk,
                      lda=M if conf.global_a_layout.col_major else K, ldb=K, ldc=M, ldd=M)
    chunks, rows = C.c_int32(0), C.c_int64(0)
    st = L.lib.gk_mgpu_host_plan(C.byref(desc), world, C.byref(chunks), C.byref(rows))
    if st != L.GK_OK:
        _raise(st)
    return chunks.value, rows.value


def broadcast_a_library(a, root: int = 0, stream=None):
    """Sends the device array `a` (its whole storage) from `root` to every rank through the library's
    communicator (gk_mgpu_broadcast, collective): the "A broadcast once" of the resident form."""
    import ctypes as C
    import torch
    from . import _lib as L
    from .matmul import _raise, handle
    dev = a.device.index
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    nbytes = a.untyped_storage().nbytes() - a.storage_offset() * a.element_size()
    with torch.cuda.device(dev):
        st = L.lib.gk_mgpu_broadcast(handle(dev), a.data_ptr(), nbytes, root, C.c_void_p(s))
    if st != L.GK_OK:
        _raise(st)
    return a


def colshard_matmul_device(conf, a, b_block, c_block, d_block, *, a_mode: str = "resident", root: int = 0,
                           k_panels: int = 0, epilogue=None, stream=None, **transforms):
    """This rank's block of the sharded product with device operands (gk_mgpu_gemm_colshard).
    `conf` describes the local block (N = this rank's columns).  a_mode "resident": A is already on
    every rank; "broadcast": rank `root` holds A and it travels to every rank's `a` in K-panels over
    NVLink while the panels that have arrived are multiplied (collective: every rank calls)."""
    import ctypes as C
    import torch
    from . import _lib as L
    from . import epilogue as Epilogue
    from . import kernel as Kernel
    from .matmul import _raise, handle, lower
    hooks = {k.replace("transform_", ""): v for k, v in transforms.items()}
    desc, epi, (pa, pb, pc, pd) = lower(conf, a, b_block, c_block, d_block, hooks, epilogue or Epilogue.Default(),
                                        Kernel.matmul_singlestage)
    dev = d_block.device.index
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    mode = {"resident": L.GK_MGPU_A_RESIDENT, "broadcast": L.GK_MGPU_A_BROADCAST}[a_mode]
    with torch.cuda.device(dev):
        st = L.lib.gk_mgpu_gemm_colshard(handle(dev), C.byref(desc), pa, mode, root, k_panels, pb, pc, pd, C.byref(epi),
                                         None, 0, C.c_void_p(s))
    if st != L.GK_OK:
        _raise(st)
    return d_block


def colshard_matmul_host(conf, a_host, b_host_block, c_host_block, d_host_block, *, epilogue=None, stream=None,
                         device_index=None, times: bool = False, **transforms):
    """The sharded product with operands and result in host memory (gk_mgpu_gemm_colshard_host,
    collective).  `a_host` is the whole A in this rank's host memory; each rank sends only 1/world of
    it over its own PCIe link and NCCL all-gathers assemble A on every GPU over NVLink while the
    rank's block of B goes up; row chunks of D are multiplied and sent back as their chunk of A
    completes.  Returns the phase times of this rank (a dict) when `times` is set."""
    import ctypes as C
    import torch
    from . import _lib as L
    from . import epilogue as Epilogue
    from . import kernel as Kernel
    from .matmul import _raise, handle, lower
    hooks = {k.replace("transform_", ""): v for k, v in transforms.items()}
    desc, epi, (pa, pb, pc, pd) = lower(conf, a_host, b_host_block, c_host_block, d_host_block, hooks,
                                        epilogue or Epilogue.Default(), Kernel.matmul_singlestage)
    dev = device_index if device_index is not None else torch.cuda.current_device()
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    t = L.MgpuTimes()
    with torch.cuda.device(dev):
        st = L.lib.gk_mgpu_gemm_colshard_host(handle(dev), C.byref(desc), pa, pb, pc, pd, C.byref(epi), C.c_void_p(s),
                                              C.byref(t) if times else None)
    if st != L.GK_OK:
        _raise(st)
    if times:
        return {f: getattr(t, f) for f, _ in L.MgpuTimes._fields_ if f != "reserved"}
    return d_host_block


def allgather_a_chunks(a_host, trans_a: bool, rank: int, world: int, chunks: int, rows: int, group=None):
    """The data movement of the host path in `torch.distributed` terms (what the CPU tests run over
    gloo; on GPUs the library does it with NCCL): A is cut into `chunks` row chunks of `rows` rows; of
    every chunk each rank contributes the 1/world share it would upload — columns [rank*K/world, ...)
    of a column-major A, rows [rank*rows_i/world, ...) of the chunk for a transposed one — and an
    all-gather assembles the chunk on every rank.  `a_host` is op(A) as an (M, K) tensor, of which only
    this rank's shares are read.  Returns the list of assembled chunks, each (rows_i, K)."""
    import torch
    import torch.distributed as dist
    M, K = a_host.shape
    out = []
    for i in range(chunks):
        i0, i1 = i * rows, min((i + 1) * rows, M)
        if not trans_a:
            kc = K // world
            mine = a_host[i0:i1, rank * kc:(rank + 1) * kc].T.contiguous()      # column-major piece (kc columns)
        else:
            mc = (i1 - i0) // world
            mine = a_host[i0 + rank * mc:i0 + (rank + 1) * mc, :].contiguous()   # stored K x M: columns of the store
        if world > 1:
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine, group=group)
        else:
            parts = [mine]
        whole = torch.cat(parts, dim=0)
        out.append(whole.T if not trans_a else whole)
    return out


def gather_columns(d_block, shard: ColumnShard, group=None):
    """Assembles the full D on every rank from the column blocks (outside any timed region; used by
    tests and by callers that want D in one place).  `d_block` is the contiguous storage of the
    rank's block, shape (count, M) for column-major data.  Returns a (n_total, M) tensor."""
    import torch
    import torch.distributed as dist
    world = shard.world
    if world == 1 or not (dist.is_available() and dist.is_initialized()):
        return d_block
    m = d_block.shape[1]
    # blocks may differ in size: exchange through padded buffers of the largest block
    sizes = [None] * world
    dist.all_gather_object(sizes, int(d_block.shape[0]), group=group)
    biggest = max(sizes)
    padded = torch.zeros(biggest, m, dtype=d_block.dtype, device=d_block.device)
    padded[: d_block.shape[0]] = d_block
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], dim=0)
