#!/usr/bin/env python
"""Benchmark of the GEMM hot path on B200: `python bench.py --gpus N --steps K --warmup W`.

Workload (config.workload): the shape the headline metric is quoted on — C = A*B with A, B
Float16 ~ U[0,1) 8192 x 8192 column-major, C Float32, alpha = 1, beta = 0 (synthetic, seeded).
One step = one such GEMM per GPU through the C ABI.  With N > 1 (one process per GPU under
torchrun) the path is sharded by column blocks of B and C: rank r owns its own 8192 columns, A is
broadcast once with NCCL before the timed region and stays resident, and no collective runs inside
a step (weak scaling: the problem is M = K = 8192, N = 8192 * ranks).

Prints one JSON line: device-timed throughput (`value`), the same metric measured end to end from
host buffers (`e2e`), the tensor-core roofline of the kernel (`roofline`) and, at N = 1, the CPU
baseline (`cpu_baseline`, numpy/OpenBLAS sgemm on the Float32-promoted inputs — the reference's
own CPU check is LinearAlgebra.mul!, i.e. OpenBLAS sgemm).

`--impl reference` times that CPU product alone (rank 0 only) for the same metric and config.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
if "reference" in sys.argv:
    # the CPU arm uses every host core: torchrun exports OMP_NUM_THREADS=1 to its workers, which would
    # pin the BLAS pool to one thread before numpy is even imported
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)
sys.path.insert(0, str(ROOT / "gemmkernels.jl_b200"))

import numpy as np  # noqa: E402

METRIC = "GEMM TFLOP/s (FP16->FP32, 8192^3)"
N_DIM = 8192
FLOPS_PER_GEMM = 2.0 * N_DIM ** 3
# DRAM traffic of one launch, from the ncu capture summarised in profiles/ (dram read + write).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1.107e9   # dram__bytes.sum.per_second (1.619 TB/s) x gpu__time_duration (683.9 us)


def measured_peaks():
    """Measured denominators written by the driver; fallback figures when the file is absent."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def workload_config(n_gpus: int) -> dict:
    cols = N_DIM // n_gpus
    return {"workload": f"c0: C=A*B, A,B Float16 U[0,1) {N_DIM}x{N_DIM} col-major, C Float32, alpha=1 beta=0"
                        + (f"; split by column blocks of B,C over {n_gpus} ranks ({cols} columns each), A resident on every rank "
                           "(broadcast once through the library, timed separately)" if n_gpus > 1 else ""),
            "m": N_DIM, "n_total": N_DIM, "n_per_gpu": cols, "k": N_DIM, "operator": "TCGen05Operator{Float16,Float32}",
            "l2": "inputs and output (512 MiB in all) are larger than L2; no flush between steps"
                  if n_gpus <= 2 else "per-GPU working set fits L2 at this N (strong scaling of a fixed 8192^3 product); no flush"}


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU check (OpenBLAS sgemm on promoted inputs), bounded sample
# ------------------------------------------------------------------------------------------------
def cpu_sgemm_sample(cols: int, reps: int, warmup: int):
    """Times D[:, :cols] = A * B[:, :cols] in float32 with every host thread BLAS will use.
    Returns (seconds per rep, flops per rep, threads)."""
    from oracle import gemm_oracle as O
    A, B = O.inputs_fp16_uniform01(0, N_DIM, cols, N_DIM)
    a32, b32 = A.astype(np.float32), B.astype(np.float32)
    threads = os.cpu_count() or 1
    import contextlib
    limit = contextlib.nullcontext()
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        limit = threadpool_limits(limits=threads, user_api="blas")      # every core, whatever the environment said
    except Exception:
        threadpool_info = None
    with limit:
        if threadpool_info is not None:
            blas = [p for p in threadpool_info() if p.get("user_api") == "blas"]
            if blas:
                threads = int(blas[0]["num_threads"])
        for _ in range(warmup):
            O.gemm(a32, b32)
        t0 = time.perf_counter()
        for _ in range(reps):
            O.gemm(a32, b32)
        dt = (time.perf_counter() - t0) / max(reps, 1)
    return dt, 2.0 * N_DIM * cols * N_DIM, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cols = 1024   # one eighth of the columns per step: a bounded sample of the same product
    dt, flops, threads = cpu_sgemm_sample(cols, args.steps, max(1, min(args.warmup, 3)))
    tf = flops / dt / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                             "sample": f"{N_DIM}x{cols}x{N_DIM} slice (first {cols} columns of D) of the 8192^3 product per step, "
                                       "numpy/OpenBLAS sgemm on Float32-promoted inputs"},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------------
# clocks during the timed region (read-only NVML sampling)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = None
            try:
                # NVML numbers all GPUs of the machine; CUDA only the visible ones: match by UUID
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
                try:
                    self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
                except Exception:
                    self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = None
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                break
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# the GPU arm
# ------------------------------------------------------------------------------------------------
def _timed(step, steps, warmup, barrier, max_over_ranks, torch):
    """W untimed steps, then `steps` steps between CUDA events on the launching stream; barrier and
    device synchronisation on both sides; max over ranks.  Returns milliseconds per step."""
    for _ in range(warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    return max_over_ranks(e0.elapsed_time(e1)) / steps


def c5_subrecord(args, world, rank, local, barrier, max_over_ranks, peaks):
    """Configuration 5 (16384^3 BFloat16 -> Float32) sharded by column blocks over the ranks: steady
    state with A resident, the one-shot time with A broadcast in K-panels under the product, the plain
    broadcast alone, and — in the same run, on rank 0 — the whole product on one GPU, which gives the
    strong-scaling efficiency without a second job.  Operands are drawn on the device (N(0, 0.02),
    seeded); one row of the result is checked against a torch FP32 product."""
    import torch
    import gemmkernels_b200 as GK
    from gemmkernels_b200 import multigpu
    n = 16384
    shard = multigpu.column_shard(n, world, rank, 512)
    n_loc = shard.count
    g = torch.Generator(device="cuda").manual_seed(1005)
    a = GK.cuarray(GK.BFloat16, n, n)
    if rank == 0:
        a.T.copy_((torch.randn(n, n, device="cuda", generator=g) * 0.02).to(torch.bfloat16))
    else:
        a.zero_()
    gb = torch.Generator(device="cuda").manual_seed(2005 + rank)
    b = GK.cuarray(GK.BFloat16, n, n_loc)
    b.T.copy_((torch.randn(n_loc, n, device="cuda", generator=gb) * 0.02).to(torch.bfloat16))
    d = GK.cuarray(GK.Float32, n, n_loc)
    conf = GK.get_config(gemm_shape=(n, n_loc, n), operator=GK.Operator.TCGen05Operator[GK.BFloat16, GK.Float32],
                         global_a_layout=GK.Layout.UnsafeAlignedColMajor[GK.BFloat16],
                         global_c_layout=GK.Layout.Zero[GK.Float32],
                         global_d_layout=GK.Layout.UnsafeAlignedColMajor[GK.Float32], block_shape=(128, 128, 64))
    steps, warm = min(args.steps, 20), 3
    rec = {"workload": f"c5: 16384^3 BFloat16 N(0,0.02) -> Float32, column blocks of B,C over {world} rank(s) "
                       f"({n_loc} columns on rank 0)", "steps": steps, "warmup": warm}
    if world > 1:
        # one-shot: A leaves rank 0 in K-panels on the communication stream while the panels that have
        # arrived are multiplied (first call also pays nothing extra: the communicator is warm by now)
        def one_shot():
            multigpu.colshard_matmul_device(conf, a, b, None, d, a_mode="broadcast", root=0)
        rec["one_shot_broadcast_overlapped_ms"] = _timed(one_shot, 3, 1, barrier, max_over_ranks, torch)
        rec["a_broadcast_alone_ms"] = _timed(lambda: multigpu.broadcast_a_library(a, root=0), 3, 1, barrier, max_over_ranks, torch)
    step = GK.bind(conf, a, b, None, d)
    ms = _timed(step, steps, warm, barrier, max_over_ranks, torch)
    GK.poll_status()
    if rank == 0:
        want = a[11:12].float() @ b.float()
        err = (torch.linalg.norm(d[11:12].double() - want.double()) / torch.linalg.norm(want.double())).item()
        if not err <= 1e-3:
            raise SystemExit(f"c5 result is wrong: normwise error {err}")
    flops = 2.0 * n ** 3
    plan = GK.query(conf, a, b, None, d)
    rec.update({"ms_per_step": ms, "tflops_total": flops / (ms * 1e-3) / 1e12,
                "tflops_per_gpu": flops / world / (ms * 1e-3) / 1e12,
                "frac_of_measured_per_gpu": flops / world / (ms * 1e-3) / 1e12 / peaks["tflops"],
                "tile": [int(plan.tile_m), int(plan.tile_n), int(plan.tile_k)], "grid": int(plan.grid)})
    if world > 1:
        del b, d
        n1_ms = None
        if rank == 0:
            b1 = GK.cuarray(GK.BFloat16, n, n); b1.T.copy_((torch.randn(n, n, device="cuda", generator=gb) * 0.02).to(torch.bfloat16))
            d1 = GK.cuarray(GK.Float32, n, n)
            conf1 = GK.get_config(gemm_shape=(n, n, n), operator=GK.Operator.TCGen05Operator[GK.BFloat16, GK.Float32],
                                  global_a_layout=GK.Layout.UnsafeAlignedColMajor[GK.BFloat16],
                                  global_c_layout=GK.Layout.Zero[GK.Float32],
                                  global_d_layout=GK.Layout.UnsafeAlignedColMajor[GK.Float32], block_shape=(128, 128, 64))
            step1 = GK.bind(conf1, a, b1, None, d1)
            for _ in range(warm):
                step1()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step1()
            e1.record(); torch.cuda.synchronize()
            n1_ms = e0.elapsed_time(e1) / steps
            del b1, d1
        barrier()
        if rank == 0:
            rec["n1_ms_per_step_same_run"] = n1_ms
            rec["efficiency_vs_n1"] = n1_ms / (world * ms)
    del a
    torch.cuda.empty_cache()
    return rec


def run_gpu(args):
    import torch
    import torch.distributed as dist

    import gemmkernels_b200 as GK
    from gemmkernels_b200 import _lib as L
    from oracle import gemm_oracle as O   # input generators and the CPU baseline leg only

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs one process per GPU: launch with torch.distributed.run --nproc-per-node N")
        args.gpus = world
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from gemmkernels_b200 import multigpu

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if world > 1:
        multigpu.init(device_index=local)       # the library's own communicator (NCCL found by dlopen)
    peaks = measured_peaks()

    # The metric's product, 8192^3 Float16 -> Float32, split by column blocks of B and C over the ranks
    # (strong scaling: the problem is fixed, every rank owns 8192 / N columns).  A is the same on every
    # rank (seeded); every rank draws its own block of B.
    m_dim = k_dim = n_total = N_DIM
    shard = multigpu.column_shard(n_total, world, rank, 512)
    n_loc = shard.count
    ET, tdt = GK.Float16, torch.float16
    A_host, _ = O.inputs_fp16_uniform01(0, m_dim, 8, k_dim)
    B_host = np.random.default_rng(2000 + rank).random((k_dim, n_loc), dtype=np.float32).astype(np.float16)
    a_pin = torch.from_numpy(np.ascontiguousarray(A_host.T)).to(tdt).pin_memory().T      # column-major, pinned
    b_pin = torch.from_numpy(np.ascontiguousarray(B_host.T)).to(tdt).pin_memory().T
    d_pin = torch.empty(n_loc, m_dim, dtype=torch.float32).pin_memory().T
    a = GK.cuarray(ET, m_dim, k_dim)
    b = GK.cuarray(ET, k_dim, n_loc); b.copy_(b_pin, non_blocking=True)
    d = GK.cuarray(GK.Float32, m_dim, n_loc)
    if rank == 0:
        a.copy_(a_pin, non_blocking=True)
    torch.cuda.synchronize()

    # the call a user makes: GemmKernels.matmul with a Config (TCGen05Operator, aligned layouts)
    conf = GK.get_config(gemm_shape=(m_dim, n_loc, k_dim), operator=GK.Operator.TCGen05Operator[ET, GK.Float32],
                         global_a_layout=GK.Layout.UnsafeAlignedColMajor[ET],
                         global_c_layout=GK.Layout.Zero[GK.Float32],
                         global_d_layout=GK.Layout.UnsafeAlignedColMajor[GK.Float32], block_shape=(128, 128, 64))
    plan = GK.query(conf, a, b, None, d)
    one_shot_ms = bcast_ms = None
    if world > 1:
        barrier()
        # A reaches the other ranks through the library: broadcast in K-panels overlapped with the product
        multigpu.colshard_matmul_device(conf, a, b, None, d, a_mode="broadcast", root=0)      # warm: NCCL's lazy set-up
        one_shot_ms = _timed(lambda: multigpu.colshard_matmul_device(conf, a, b, None, d, a_mode="broadcast", root=0),
                             3, 1, barrier, max_over_ranks, torch)
        bcast_ms = _timed(lambda: multigpu.broadcast_a_library(a, root=0), 3, 1, barrier, max_over_ranks, torch)

    def step():
        GK.matmul(conf, a, b, None, d, kernel=GK.Kernel.matmul_pipelined)

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    GK.poll_status()
    ms_per_step = total_ms / args.steps
    value = FLOPS_PER_GEMM / (ms_per_step * 1e-3) / 1e12

    # correctness spot check of the timed result (one row against the oracle's product)
    row = np.asarray(A_host[7:8].astype(np.float32) @ B_host.astype(np.float32))
    err = O.normwise_error(d[7:8].cpu().numpy(), row)
    if not err <= 1e-3:
        raise SystemExit(f"bench result is wrong on rank {rank}: normwise error {err}")

    # the library GEMM (cuBLAS through torch.matmul) on the same operands, same warm-up and steps, right
    # after the timed region: the comparator the reference's own benchmark runner always prints
    cublas_ms = None
    if world == 1:
        bt, at = b.T, a.T                      # contiguous views: (B^T A^T) = D^T is the row-major image of D
        cublas_out = "f32"
        try:
            torch.mm(bt, at, out_dtype=torch.float32)
            def cublas_step():
                torch.mm(bt, at, out_dtype=torch.float32)
        except Exception:
            cublas_out = "f16"                 # this torch cannot ask cuBLAS for a Float32 result: half the output bytes
            def cublas_step():
                torch.mm(bt, at)
        cublas_ms = _timed(cublas_step, args.steps, warm, barrier, max_over_ranks, torch)

    # end to end: the same product from pinned host buffers (H2D of the operands, D2H of D inside the
    # timed region, every step).  One rank: gk_gemm_host.  Several: every rank uploads 1/N of A over its
    # own PCIe link, NCCL all-gathers assemble A over NVLink, its block of B goes up and its block of D
    # comes back (gk_mgpu_gemm_colshard_host).
    phases = None
    if world > 1:
        def e2e_step():
            return multigpu.colshard_matmul_host(conf, a_pin, b_pin, None, d_pin, device_index=local, times=True)
    else:
        def e2e_step():
            GK.matmul_host(conf, a_pin, b_pin, None, d_pin, device_index=local)
    for _ in range(2):
        e2e_step()
    barrier()
    e2e_steps = min(args.steps, 100)   # ~10 ms per step over PCIe on one GPU: bounded so the default run stays short
    acc = {}
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        t = e2e_step()
        if t:
            for k, v in t.items():
                acc[k] = acc.get(k, 0.0) + float(v)
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
    err = O.normwise_error(d_pin[7:8].numpy(), row)
    if not err <= 1e-3:
        raise SystemExit(f"end-to-end result is wrong on rank {rank}: normwise error {err}")
    e2e_value = FLOPS_PER_GEMM / (e2e_ms * 1e-3) / 1e12
    if world > 1:
        phases = {k: acc[k] / e2e_steps for k in ("upload_ms", "collective_ms", "compute_ms", "download_ms", "total_ms")}
        phases_max = {k: max_over_ranks(v) for k, v in phases.items()}
        tot = torch.tensor([acc["h2d_bytes"] / e2e_steps, acc["d2h_bytes"] / e2e_steps], device="cuda", dtype=torch.float64)
        dist.all_reduce(tot)
        all_h2d, all_d2h = float(tot[0].item()), float(tot[1].item())
        h2d = int(acc["h2d_bytes"] / e2e_steps); d2h = int(acc["d2h_bytes"] / e2e_steps)
        chunks = int(acc["chunks"] / e2e_steps)
    else:
        h2d = a_pin.numel() * 2 + b_pin.numel() * 2
        d2h = d_pin.numel() * 4
    del a, b, d
    torch.cuda.empty_cache()

    c5 = None if args.no_c5 else c5_subrecord(args, world, rank, local, barrier, max_over_ranks, peaks)

    if rank != 0:
        if world > 1:
            dist.barrier(); multigpu.shutdown(local); dist.destroy_process_group()
        return 0

    achieved = FLOPS_PER_GEMM / world / (ms_per_step * 1e-3) / 1e12     # per launch, one GPU (rank 0's block)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(world),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps},
        "gpu_launches": args.steps,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tflops"],
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
                     "traffic_source": "ncu capture of this kernel on this shape (profiles/tc_gemm_kernel_c0_8192_fp16.md), "
                                       "not measured in this run",
                     "peak_source": f"{peaks['source']} cuBLAS bf16 burst; sustained {peaks['tflops_sustained']}",
                     "frac_of_nominal_dense_2250": achieved / 2250.0},
        "kernel": {"family": int(plan.kernel), "grid": int(plan.grid), "cluster": int(plan.cluster),
                   "tile": [int(plan.tile_m), int(plan.tile_n), int(plan.tile_k)], "stages": int(plan.stages),
                   "smem_bytes": int(plan.smem_bytes), "tmem_columns": int(plan.tmem_columns)},
    }
    if cublas_ms is not None:
        line["cublas_same_run_tflops"] = FLOPS_PER_GEMM / (cublas_ms * 1e-3) / 1e12
        line["vs_cublas_same_run"] = cublas_ms / ms_per_step
        line["cublas_out_dtype"] = cublas_out
    if world > 1:
        tm_, tn_ = int(plan.tile_m), int(plan.tile_n)
        tiles = (-(-m_dim // tm_)) * (-(-n_loc // tn_))
        slots = max(1, torch.cuda.get_device_properties(local).multi_processor_count // int(plan.cluster))
        rounds = -(-tiles // slots)
        line["a_broadcast_ms"] = bcast_ms
        line["one_shot_broadcast_overlapped_ms"] = one_shot_ms
        line["e2e"]["phases_ms_rank0"] = phases
        line["e2e"]["phases_ms_max_over_ranks"] = phases_max
        line["e2e"]["a_chunks"] = chunks
        line["e2e"]["h2d_gbs_per_rank"] = h2d / (phases["upload_ms"] * 1e-3) / 1e9 if phases["upload_ms"] > 0 else None
        line["e2e"]["d2h_gbs_per_rank"] = d2h / (phases["download_ms"] * 1e-3) / 1e9 if phases["download_ms"] > 0 else None
        line["e2e"]["all_ranks_h2d_bytes_per_step"] = all_h2d
        line["e2e"]["all_ranks_d2h_bytes_per_step"] = all_d2h
        line["e2e"]["host_link_gbs_all_ranks"] = (all_h2d + all_d2h) / (e2e_ms * 1e-3) / 1e9
        line["e2e"]["limiter"] = ("the host: A and B go up once (1/N of A per rank) and D comes down once whatever N is, and the "
                                  "ranks' copies share the host's memory and PCIe root ports; host_link_gbs_all_ranks is what "
                                  "they sustained together (one GPU alone: ~72 GB/s over both directions)")
        line["limiter"] = (f"each rank's block is {tiles} tiles of {tm_}x{tn_} on {slots} CTA slots = {rounds} round(s) "
                           f"{tiles / (rounds * slots):.0%} full (one GPU alone: "
                           f"{(N_DIM // 256) * (N_DIM // 512)} tiles of 256x512 on 74 slots, 99% full)"
                           + ("; the single accumulator stage of the 512-wide tile leaves each tile's epilogue exposed" if tn_ == 512 else ""))
    if c5 is not None:
        line["c5"] = c5
    if world == 1 and not args.no_cpu_baseline:
        cols = 2048
        dt, flops, threads = cpu_sgemm_sample(cols, 3, 1)
        line["cpu_baseline"] = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": f"{N_DIM}x{cols}x{N_DIM} slice of the 8192^3 product, 3 timed runs after 1 warm-up, "
                                          "numpy/OpenBLAS sgemm on Float32-promoted inputs"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(); multigpu.shutdown(local); dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------------------------------------
# the other configurations, kernel-only (one GPU): parity cases first, timed here for the record
# ------------------------------------------------------------------------------------------------
def run_side(args):
    """c1 2048^3 FP16; c2 4096^3 FP32 FFMA, A transposed, bias(M)+ReLU; c3 4096^3 planar complex FP16;
    c4 the contraction C[a,b,c,d] = sum A[a,e,b,f] B[d,f,c,e], extents 32; diag 4096^2 diagonal A.
    Inputs are drawn on the device (torch RNG) and stay resident; no end-to-end leg, no CPU leg.
    A sample of the timed result is checked against a torch FP32 product of the same operands."""
    import torch

    import gemmkernels_b200 as GK
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(7)
    Lay, Op = GK.Layout, GK.Operator

    def rnd(et, *shape, lo=0.0, hi=1.0):
        t = GK.cuarray(et, *shape)
        t.copy_((torch.rand(tuple(reversed(shape)), device="cuda", generator=g) * (hi - lo) + lo).permute(*reversed(range(len(shape)))))
        return t

    w = args.workload
    bound, unit = "tensor", "TFLOP/s"
    if w == "c1":
        n = 2048
        a, b, d = rnd(GK.Float16, n, n), rnd(GK.Float16, n, n), GK.cuarray(GK.Float32, n, n)
        conf = GK.get_config(gemm_shape=(n, n, n), operator=Op.TCGen05Operator[GK.Float16, GK.Float32],
                             global_a_layout=Lay.UnsafeAlignedColMajor[GK.Float16], global_c_layout=Lay.Zero[GK.Float32],
                             global_d_layout=Lay.UnsafeAlignedColMajor[GK.Float32])
        step = GK.bind(conf, a, b, None, d)
        check = lambda: (d[5:9], a[5:9].float() @ b.float())
        flops, name = 2.0 * n ** 3, "c1: 2048^3 Float16 -> Float32, col-major, tcgen05"
        plan = GK.query(conf, a, b, None, d)
    elif w == "c2":
        n = 4096
        a, b, d = rnd(GK.Float32, n, n, lo=-1), rnd(GK.Float32, n, n, lo=-1), GK.cuarray(GK.Float32, n, n)
        bias = torch.rand(n, device="cuda", generator=g) - 0.5
        conf = GK.get_config(gemm_shape=(n, n, n), operator=Op.FPUOp[8, 8, 1, 4, 8, 1, GK.Float32, GK.Float32],
                             global_a_layout=Lay.UnsafeAlignedRowMajor[GK.Float32],
                             global_b_layout=Lay.UnsafeAlignedColMajor[GK.Float32], global_c_layout=Lay.Zero[GK.Float32],
                             global_d_layout=Lay.UnsafeAlignedColMajor[GK.Float32])
        epi = GK.Epilogue.Bias(bias, axis="row")
        step = GK.bind(conf, a, b, None, d, epilogue=epi, transform_shared_to_global_d=GK.Transform.ReLU())
        check = lambda: (d[5:9], torch.relu(a[:, 5:9].t().double() @ b.double() + bias[5:9, None].double()).float())
        flops, name, bound = 2.0 * n ** 3, "c2: 4096^3 Float32 FFMA, A transposed, bias(M)+ReLU fused", "fp32-fma"
        plan = GK.query(conf, a, b, None, d, epilogue=epi, transform_shared_to_global_d=GK.Transform.ReLU())
    elif w == "c3":
        n = 4096
        a, b = rnd(GK.Float16, n, n, 2, lo=-1), rnd(GK.Float16, n, n, 2, lo=-1)
        d = GK.cuarray(GK.Float32, n, n, 2)
        conf = GK.get_config(gemm_shape=(n, n, n), operator=Op.WMMAComplexOp[16, 16, 16, GK.Float16, GK.Float32],
                             global_a_layout=Lay.SplitColMajor[GK.Float16], global_c_layout=Lay.Zero[GK.Float32],
                             global_d_layout=Lay.SplitColMajor[GK.Float32], block_shape=(64, 64, 32))
        step = GK.bind(conf, a, b, None, d)
        def check():
            ar, ai, br, bi = a[5:9, :, 0].float(), a[5:9, :, 1].float(), b[..., 0].float(), b[..., 1].float()
            return d[5:9], torch.stack([ar @ br - ai @ bi, ar @ bi + ai @ br], dim=-1)
        flops, name = 8.0 * n ** 3, "c3: 4096^3 planar Complex{Float16} -> Complex{Float32} (8 N^3 real flops), tcgen05"
        plan = GK.query(conf, a, b, None, d)
    elif w == "c4":
        e = 32
        a, b = rnd(GK.Float16, e, e, e, e, lo=-1), rnd(GK.Float16, e, e, e, e, lo=-1)
        d = GK.cuarray(GK.Float32, e, e, e, e)
        step = GK.bind_contract(d, "abcd", a, "aebf", b, "dfce")
        check = lambda: (d[3], torch.einsum("ebf,dfce->bcd", a[3].float(), b.float()))
        flops, name = 2.0 * e ** 6, "c4: C[a,b,c,d] = sum_ef A[a,e,b,f] B[d,f,c,e], extents 32 (M=N=K=1024), tcgen05 via 5-D TMA"
        plan = GK.contract_query(d, "abcd", a, "aebf", b, "dfce")
    elif w == "c5":
        n = 16384
        a, b, d = rnd(GK.BFloat16, n, n, lo=-0.03, hi=0.03), rnd(GK.BFloat16, n, n, lo=-0.03, hi=0.03), GK.cuarray(GK.Float32, n, n)
        conf = GK.get_config(gemm_shape=(n, n, n), operator=Op.TCGen05Operator[GK.BFloat16, GK.Float32],
                             global_a_layout=Lay.UnsafeAlignedColMajor[GK.BFloat16], global_c_layout=Lay.Zero[GK.Float32],
                             global_d_layout=Lay.UnsafeAlignedColMajor[GK.Float32])
        step = GK.bind(conf, a, b, None, d)
        check = lambda: (d[5:9], a[5:9].float() @ b.float())
        flops, name = 2.0 * n ** 3, "c5 on one GPU: 16384^3 BFloat16 -> Float32, col-major, tcgen05"
        plan = GK.query(conf, a, b, None, d)
    else:
        # diag: 4096^2 (the reference's benchmark size; 160 MiB working set, partly L2-resident);
        # diag-large: 16384 x 8192 columns (1.25 GiB streamed: 10x L2, a clean HBM figure)
        n = 4096 if w == "diag" else 16384
        cols = n if w == "diag" else 8192
        v, b, c, d = rnd(GK.Float16, n), rnd(GK.Float16, n, cols), rnd(GK.Float32, n, cols), GK.cuarray(GK.Float32, n, cols)
        conf = GK.get_config(gemm_shape=(n, cols, n), operator=Op.TCGen05Operator[GK.Float16, GK.Float32],
                             global_a_layout=Lay.Diagonal[GK.Float16], global_b_layout=Lay.UnsafeAlignedColMajor[GK.Float16],
                             global_c_layout=Lay.UnsafeAlignedColMajor[GK.Float32], block_shape=(128, 128, 64),
                             shared_a_layout=Lay.Padded[Lay.UnsafeAlignedColMajor[GK.Float16], 8])
        step = GK.bind(conf, v, b, c, d)
        check = lambda: (d[5:9], v[5:9, None].float() * b[5:9].float() + c[5:9])
        # streams B (2 B), C (4 B) in and D (4 B) out per element
        flops, name, bound, unit = 10.0 * n * cols, f"{w}: D = diag(v) B + C, {n}x{cols}, Float16 B, Float32 C/D (10 B per element)", "hbm", "GB/s"
        plan = GK.query(conf, v, b, c, d)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    GK.poll_status()
    ms = e0.elapsed_time(e1) / args.steps
    got, want = check()
    err = (torch.linalg.norm(got.double() - want.double()) / torch.linalg.norm(want.double())).item()
    if not err <= 1e-3:
        raise SystemExit(f"bench result is wrong: normwise error {err}")
    peaks = measured_peaks()
    scale = 1e9 if bound == "hbm" else 1e12
    achieved = flops / (ms * 1e-3) / scale
    if bound == "tensor":
        peak, src = peaks["tflops"], f"{peaks['source']} cuBLAS bf16 burst"
    elif bound == "hbm":
        peak, src = peaks["hbm_gbs"], f"{peaks['source']} copy bandwidth"
    else:
        import ctypes as C
        from gemmkernels_b200 import _lib as L
        sm = torch.cuda.get_device_properties(0).multi_processor_count
        mhz = clocks.get("sm_max_mhz") or 1965
        nominal = sm * 128 * 2 * mhz * 1e6 / 1e12
        measured = C.c_double(0.0)
        st = L.lib.gk_measure_fp32_fma(GK.handle(0), C.byref(measured), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if st != 0:
            raise SystemExit(f"FMA peak measurement failed: {L.lib.gk_last_error_message()}")
        peak = measured.value
        src = (f"measured here: register-only packed-FMA kernel (gk_measure_fp32_fma); "
               f"nominal {nominal:.1f} = {sm} SMs x 128 FMA lanes x 2 x {mhz} MHz")
    print(json.dumps({
        "metric": f"{unit} ({name})", "value": achieved, "unit": unit, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"c2": "f32", "diag": "f32", "diag-large": "f32", "c5": "bf16"}.get(w, "f16"), "data": "synthetic",
        "config": {"workload": name, "l2": "back-to-back launches on resident operands; kernel-only, no end-to-end leg"},
        "clocks": clocks, "gpu_launches": args.steps, "sample_normwise_error": err,
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                     "traffic": None, "peak_source": src},
        "us_per_launch": ms * 1e3,
        **({"hbm_gbs_of_algorithmic_bytes": (3 * 4096 * 4096 * 4 + 4096 * 4) / (ms * 1e-3) / 1e9} if w == "c2" else {}),
        "kernel": {"family": int(plan.kernel), "grid": int(plan.grid), "cluster": int(plan.cluster),
                   "tile": [int(plan.tile_m), int(plan.tile_n), int(plan.tile_k)], "stages": int(plan.stages),
                   "smem_bytes": int(plan.smem_bytes), "tmem_columns": int(plan.tmem_columns)},
    }), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c5", action="store_true", help="skip the 16384^3 BFloat16 sub-record")
    ap.add_argument("--workload", default="c0", choices=["c0", "c1", "c2", "c3", "c4", "c5", "diag", "diag-large"],
                    help="c0: the headline 8192^3 FP16 GEMM, split by column blocks over the ranks, with the 16384^3 "
                         "BF16 configuration as a sub-record of the same line; c1-c4, diag: the other "
                         "configurations (c5: on one GPU; diag-large: 16384 x 8192, ten times L2), kernel-only on one GPU")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload != "c0":
        return run_side(args)
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
