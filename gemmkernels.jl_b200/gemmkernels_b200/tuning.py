"""Autotuner for the tcgen05 GEMM on B200: sweeps tile width, CTA pairing, pipeline depth and raster
band per problem, through the C ABI, timing with CUDA events.

Mirrors what tuning/tune.jl of the reference does where it still applies:
  * a parameter sweep per (shape, transposes) — there: block/warp/operator shapes (tuning/wmma.jl:34-47);
    here: tile_n, cta_group, stages, raster_group;
  * "measure until no improvement" timing (tuning/tune.jl:143-163);
  * each candidate's result is verified against an independent product (tune.jl:172-176 compares with
    the cuBLAS baseline) — here sampled rows of a Float32 `torch.matmul` of the same operands;
  * the winners become the defaults: `emit_table` writes them as the table compiled into the library
    (csrc/tuned_table.inc), `load_into_library` hands them to a running library (gk_load_tuning), and
    the planner consults both before its own cost model (tuning/wmma.jl:34-47 plays this role there);
  * an error taxonomy per candidate (tune.jl:90-179): config_error / cuda_error / invalid_result / timeout;
  * checkpoint and resume (tune.jl:315-357): one JSON line per measured candidate, measured keys are
    skipped on restart, unreadable lines are ignored;
  * waiting out thermal throttling before a measurement (tune.jl:223-247), with read-only NVML.
Locking GPU clocks (tuning/setup.sh:29-43) changes a setting that outlasts the process; `lock_clocks`
exists for machines where the operator wants it, is never called by the tuner itself, and is off by
default.
"""
from __future__ import annotations

import itertools
import json
import os
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable, Iterable, Iterator

TILE_N = (64, 128, 192, 256, 512)   # 512 = two 256-column accumulators sharing each A stage (CTA pairs only)
CTA_GROUP = (1, 2)
STAGES = (0, 3, 4, 6)          # 0 = as many as shared memory holds
RASTER_GROUP = (0, 4, 8, 16)   # 0 = built-in choice
K_BLOCKS_PER_STAGE = (1, 2)    # 128-byte k-blocks per pipeline stage


@dataclass(frozen=True)
class Problem:
    m: int
    n: int
    k: int
    trans_a: bool = False
    trans_b: bool = False
    dtype: str = "Float16"      # Float16 | BFloat16 | TF32
    with_c: bool = False        # D = A*B + C (C Float32) instead of D = A*B

    def key(self) -> str:
        return (f"{self.dtype}:{self.m}x{self.n}x{self.k}:{'T' if self.trans_a else 'N'}{'T' if self.trans_b else 'N'}"
                + ("+C" if self.with_c else ""))


@dataclass(frozen=True)
class Candidate:
    tile_n: int
    cta_group: int
    stages: int
    raster_group: int
    k_blocks_per_stage: int = 0

    def key(self) -> str:
        base = f"tn{self.tile_n}-cg{self.cta_group}-st{self.stages}-rg{self.raster_group}"
        return base + (f"-kps{self.k_blocks_per_stage}" if self.k_blocks_per_stage else "")


def candidates(problem: Problem, tile_n=TILE_N, cta_group=CTA_GROUP, stages=STAGES,
               raster_group=RASTER_GROUP, k_blocks_per_stage=K_BLOCKS_PER_STAGE) -> Iterator[Candidate]:
    """The sweep for one problem, without the combinations the engine would refuse anyway."""
    for tn, cg, st, rg, kps in itertools.product(tile_n, cta_group, stages, raster_group, k_blocks_per_stage):
        if cg == 2 and tn % 64:
            continue
        if tn == 512 and cg != 2:
            continue
        if tn > max(64, -(-problem.n // 32) * 32):        # wider than the whole matrix: a duplicate
            continue
        yield Candidate(tn, cg, st, rg, kps)
    yield Candidate(0, 0, 0, 0)                            # the built-in choice, for comparison


# ------------------------------------------------------------------------------------------------
# results file: JSON lines, append-only
# ------------------------------------------------------------------------------------------------
def load_results(path) -> dict:
    """(problem key, candidate key) -> record.  Lines that do not parse are skipped, as a run killed
    mid-write leaves at most one such line."""
    out = {}
    p = Path(path)
    if not p.exists():
        return out
    for line in p.read_text().splitlines():
        try:
            rec = json.loads(line)
            out[(rec["problem"], rec["candidate"])] = rec
        except (ValueError, KeyError):
            continue
    return out


def append_result(path, rec: dict) -> None:
    """Appends one line; a torn last line (no newline) is closed first so the new record stays readable."""
    torn = False
    if os.path.exists(path) and os.path.getsize(path):
        with open(path, "rb") as f:
            f.seek(-1, os.SEEK_END)
            torn = f.read(1) != b"\n"
    with open(path, "a") as f:
        f.write(("\n" if torn else "") + json.dumps(rec) + "\n")
        f.flush()
        os.fsync(f.fileno())


def best(results: dict, problem: Problem):
    """Fastest successful record of a problem, or None."""
    ok = [r for (pk, _), r in results.items() if pk == problem.key() and r.get("category") == "success"]
    return min(ok, key=lambda r: r["time_us"]) if ok else None


# ------------------------------------------------------------------------------------------------
# timing: repeat batches until the minimum stops improving
# ------------------------------------------------------------------------------------------------
def measure_until_stable(run_batch: Callable[[int], float], batch: int = 10, patience: int = 3,
                         max_batches: int = 50, rel_improvement: float = 0.002) -> float:
    """`run_batch(n)` returns the mean time of n back-to-back launches (any unit).  Batches are
    repeated until `patience` in a row fail to beat the best by `rel_improvement`."""
    best_t = float("inf")
    stale = 0
    for _ in range(max_batches):
        t = run_batch(batch)
        if t < best_t * (1.0 - rel_improvement):
            best_t, stale = t, 0
        else:
            best_t = min(best_t, t)
            stale += 1
            if stale >= patience:
                break
    return best_t


# ------------------------------------------------------------------------------------------------
# NVML (read-only): wait while the GPU is thermally throttled
# ------------------------------------------------------------------------------------------------
THERMAL_BITS = 0x8 | 0x20 | 0x40     # hw_slowdown | sw_thermal_slowdown | hw_thermal_slowdown


def wait_if_throttled(nvml, handle, max_wait_s: float = 30.0, poll_s: float = 0.5, sleep=time.sleep) -> bool:
    """Returns True once no thermal reason is active (False if `max_wait_s` ran out)."""
    waited = 0.0
    while True:
        try:
            mask = nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
        except AttributeError:
            mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
        if not (mask & THERMAL_BITS):
            return True
        if waited >= max_wait_s:
            return False
        sleep(poll_s)
        waited += poll_s


def lock_clocks(nvml, handle, sm_mhz: int, *, i_understand_this_outlasts_the_process: bool = False) -> None:
    """What tuning/setup.sh does with `nvidia-smi -lgc`.  Never called by this module; refuses unless
    the caller states that the setting persists after the process (it needs root, and the next user
    of the GPU inherits it).  Pair with `nvmlDeviceResetGpuLockedClocks`."""
    if not i_understand_this_outlasts_the_process:
        raise PermissionError("locking clocks changes a GPU setting that outlasts this process; not done by default")
    nvml.nvmlDeviceSetGpuLockedClocks(handle, sm_mhz, sm_mhz)


# ------------------------------------------------------------------------------------------------
# the sweep
# ------------------------------------------------------------------------------------------------
def tune(problems: Iterable[Problem], results_path, *, measure: Callable[[Problem, Candidate | None], dict] | None = None,
         candidate_fn=candidates, log=print) -> dict:
    """Measures every candidate of every problem that the results file does not hold yet.
    `measure(problem, candidate)` returns {"category": ..., "time_us": ...}; it defaults to the GPU
    measurement below.  Returns the results dictionary."""
    measure = measure or gpu_measure
    results = load_results(results_path)
    for prob in problems:
        for cand in candidate_fn(prob):
            k = (prob.key(), cand.key())
            if k in results:
                continue
            try:
                rec = measure(prob, cand)
            except Exception as e:     # a candidate must never take the sweep down
                rec = {"category": "unknown_error", "message": str(e)[:200]}
            rec.update(problem=prob.key(), candidate=cand.key(), **asdict(cand))
            append_result(results_path, rec)
            results[k] = rec
            log(f"{prob.key()} {cand.key()}: {rec['category']}" + (f" {rec['time_us']:.1f} us" if "time_us" in rec else ""))
        b = best(results, prob)
        if b:
            flops = 2.0 * prob.m * prob.n * prob.k
            log(f"best for {prob.key()}: {b['candidate']} {b['time_us']:.1f} us = {flops / b['time_us'] / 1e6:.0f} TFLOP/s")
    return results


# ------------------------------------------------------------------------------------------------
# one candidate on the GPU
# ------------------------------------------------------------------------------------------------
_ELTYPES = {"Float16": "Float16", "BFloat16": "BFloat16", "TF32": "Float32"}
_cache: dict = {}


def _operands(prob: Problem):
    """Seeded operands and the built-in configuration's output, made once per problem."""
    import torch
    from . import eltypes, arrays
    if prob.key() in _cache:
        return _cache[prob.key()]
    _cache.clear()                                     # one problem resident at a time
    et = getattr(eltypes, _ELTYPES[prob.dtype])
    g = torch.Generator(device="cuda").manual_seed(1234)
    def rnd(r, c):
        t = arrays.cuarray(et, r, c)
        t.copy_((torch.rand(c, r, device="cuda", generator=g) - 0.5).t())
        return t
    a = rnd(*((prob.k, prob.m) if prob.trans_a else (prob.m, prob.k)))
    b = rnd(*((prob.n, prob.k) if prob.trans_b else (prob.k, prob.n)))
    c = None
    if prob.with_c:
        c = arrays.cuarray(eltypes.Float32, prob.m, prob.n)
        c.copy_(torch.rand(prob.n, prob.m, device="cuda", generator=g).t())
    d = arrays.cuarray(eltypes.Float32, prob.m, prob.n)
    # the comparator: sampled rows of the product, computed by the library GEMM of torch in Float32
    # (for TF32 problems on the operands as the tensor cores read them: low 13 mantissa bits cleared)
    rows = torch.randperm(prob.m, device="cuda", generator=g)[: min(prob.m, 64)].sort().values
    def as_read(t):
        t = t.float()
        return (t.view(torch.int32) & -8192).view(torch.float32) if prob.dtype == "TF32" else t
    opa = as_read(a).t() if prob.trans_a else as_read(a)
    opb = as_read(b).t() if prob.trans_b else as_read(b)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        want = opa[rows] @ opb
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    if c is not None:
        want = want + c[rows]
    _cache[prob.key()] = (a, b, c, d, rows, want)
    return _cache[prob.key()]


def _config(prob: Problem, cand: Candidate | None):
    from . import eltypes, layout as Layout, operator as Operator
    from .config import get_config
    et = getattr(eltypes, _ELTYPES[prob.dtype])
    la = Layout.UnsafeAlignedRowMajor[et] if prob.trans_a else Layout.UnsafeAlignedColMajor[et]
    lb = Layout.UnsafeAlignedRowMajor[et] if prob.trans_b else Layout.UnsafeAlignedColMajor[et]
    extra = {} if cand is None else dict(tile_n=cand.tile_n, cta_group=cand.cta_group, stages=cand.stages,
                                         raster_group=cand.raster_group, k_blocks_per_stage=cand.k_blocks_per_stage)
    return get_config(gemm_shape=dict(M=prob.m, N=prob.n, K=prob.k),
                      operator=Operator.TCGen05Operator[Operator.TF32 if prob.dtype == "TF32" else et, eltypes.Float32],
                      global_a_layout=la, global_b_layout=lb,
                      global_c_layout=(Layout.UnsafeAlignedColMajor if prob.with_c else Layout.Zero)[eltypes.Float32],
                      global_d_layout=Layout.UnsafeAlignedColMajor[eltypes.Float32], **extra)


def gpu_measure(prob: Problem, cand: Candidate, *, rtol: float = 1e-3, nvml=None, nvml_handle=None) -> dict:
    """Verifies and times one candidate.  Categories: success, config_error (the engine refused the
    combination), invalid_result (sampled rows differ from the Float32 torch.matmul of the same
    operands), timeout (a device-side wait gave up), cuda_error (anything else the library reported)."""
    import torch
    from .config import ConfigError
    from .matmul import bind, matmul, poll_status, DeviceTimeout, GemmKernelsError
    a, b, c, d, rows, want = _operands(prob)
    try:
        conf = _config(prob, cand)
        d.zero_()
        from .matmul import query
        plan = query(conf, a, b, c, d)          # what the library resolves this candidate to
        resolved = {"plan_tile_n": int(plan.tile_n), "plan_cta_group": int(plan.cluster), "plan_stages": int(plan.stages),
                    "plan_tile_k": int(plan.tile_k)}
        launch = bind(conf, a, b, c, d)
        launch()
        torch.cuda.synchronize()
        poll_status()
    except ConfigError as e:
        return {"category": "config_error", "message": str(e)[:200]}
    except DeviceTimeout as e:
        return {"category": "timeout", "message": str(e)[:200]}
    except GemmKernelsError as e:
        return {"category": "cuda_error", "message": str(e)[:200]}
    err = (torch.linalg.norm(d[rows].double() - want.double()) / torch.linalg.norm(want.double()).clamp_min(1e-30)).item()
    if not err <= rtol:
        return {"category": "invalid_result", "rel_error": err}
    if nvml is not None:
        wait_if_throttled(nvml, nvml_handle)

    def run_batch(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            launch()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n

    run_batch(3)
    t = measure_until_stable(run_batch)
    poll_status()
    return {"category": "success", "time_us": t, "rel_error": err,
            "tflops": 2.0 * prob.m * prob.n * prob.k / t / 1e6, **resolved}


# ------------------------------------------------------------------------------------------------
# winners -> defaults
# ------------------------------------------------------------------------------------------------
_GK_DTYPE = {"Float16": 0, "BFloat16": 1, "TF32": 2}       # gk_dtype of the stored operands


def _parse_problem_key(key: str):
    """'Float16:2048x2048x2048:NT+C' -> (dtype, m, n, k, trans_a, trans_b, has_c)."""
    dtype, shape, rest = key.split(":")
    m, n, k = (int(x) for x in shape.split("x"))
    has_c = rest.endswith("+C")
    lay = rest[:2]
    return dtype, m, n, k, lay[0] == "T", lay[1] == "T", has_c


def winners(results: dict, min_gain: float = 0.02) -> list[dict]:
    """One entry per measured problem whose fastest candidate beats the planner's own choice (the
    candidate tn0-cg0-st0-rg0 of the same sweep) by at least `min_gain`; problems where the planner
    was already within that margin need no entry."""
    by_problem: dict = {}
    for (pk, _), r in results.items():
        if r.get("category") == "success":
            by_problem.setdefault(pk, []).append(r)
    out = []
    for pk, recs in sorted(by_problem.items()):
        top = min(recs, key=lambda r: r["time_us"])
        base = next((r for r in recs if r["candidate"] == "tn0-cg0-st0-rg0"), None)
        if top["tile_n"] == 0 or (base is not None and base["time_us"] <= top["time_us"] * (1.0 + min_gain)):
            continue
        if base is not None and "plan_tile_n" in base and "plan_tile_n" in top and all(
                base.get(f) == top.get(f) for f in ("plan_tile_n", "plan_cta_group", "plan_stages", "plan_tile_k")):
            continue                      # the winner is what the planner resolves to anyway: the gap is noise
        dtype, m, n, k, ta, tb, has_c = _parse_problem_key(pk)
        out.append(dict(dtype=_GK_DTYPE[dtype], trans_a=int(ta), trans_b=int(tb), has_c=int(has_c), m=m, n=n, k=k,
                        tile_n=top["tile_n"], cta_group=top["cta_group"], stages=top["stages"],
                        raster_group=top["raster_group"], k_blocks_per_stage=top.get("k_blocks_per_stage", 0), reserved=0,
                        time_us=top["time_us"],
                        planner_time_us=base["time_us"] if base else None, problem=pk))
    return out


def emit_table(results_path, out_path) -> int:
    """Writes the winners of a results file as the initialiser list the library compiles in
    (csrc/tuned_table.inc).  Returns the number of entries."""
    results = load_results(results_path)
    entries = winners(results)
    n_ok = sum(1 for r in results.values() if r.get("category") == "success")
    n_problems = len({pk for pk, _ in results})
    lines = ["// Generated by `python -m gemmkernels_b200.tuning --emit-table` from a sweep on B200: the fastest verified",
             "// candidate of each measured problem where it beat the planner's own choice by 2 % or more.",
             f"// This sweep: {n_problems} problems, {n_ok} verified candidates, {len(entries)} entries.",
             "// {dtype, trans_a, trans_b, has_c, m, n, k, tile_n, cta_group, stages, raster_group, k_blocks_per_stage, 0}"]
    for e in entries:
        note = f"{e['time_us']:.1f} us" + (f" (planner {e['planner_time_us']:.1f} us)" if e["planner_time_us"] else "")
        lines.append(f"    {{{e['dtype']}, {e['trans_a']}, {e['trans_b']}, {e['has_c']}, {e['m']}, {e['n']}, {e['k']}, "
                     f"{e['tile_n']}, {e['cta_group']}, {e['stages']}, {e['raster_group']}, {e['k_blocks_per_stage']}, 0}},"
                     f"   // {e['problem']}: {note}")
    Path(out_path).write_text("\n".join(lines) + "\n")
    return len(entries)


def load_into_library(results_path, device_index=None) -> int:
    """Hands the winners of a results file to the running library (gk_load_tuning) for this device:
    from then on descriptors that leave the tile to the library get the measured choice."""
    import ctypes as C
    from . import _lib as L
    from .matmul import _raise, handle
    entries = winners(load_results(results_path))
    arr = (L.TuningEntry * max(len(entries), 1))()
    for i, e in enumerate(entries):
        for f, _ in L.TuningEntry._fields_:
            setattr(arr[i], f, e[f])
    st = L.lib.gk_load_tuning(handle(device_index), arr, len(entries))
    if st != L.GK_OK:
        _raise(st)
    return len(entries)


DEFAULT_PROBLEMS = tuple(Problem(n, n, n, ta, tb) for n in (2048, 4096, 8192)
                         for ta in (False, True) for tb in (False, True))


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="Sweep the tcgen05 GEMM's tile parameters on this GPU.")
    ap.add_argument("--out", default="tuning_results.jsonl")
    ap.add_argument("--sizes", type=int, nargs="*", default=[2048, 4096, 8192])
    ap.add_argument("--shapes", nargs="*", default=[], metavar="MxNxK",
                    help="rectangular problems on top of --sizes, e.g. 8192x1024x8192 (a rank's column block)")
    ap.add_argument("--dtype", default="Float16", choices=sorted(_ELTYPES))
    ap.add_argument("--layouts", nargs="*", default=["NN", "NT", "TN", "TT"])
    ap.add_argument("--with-c", action="store_true", help="tune D = A*B + C instead of D = A*B")
    ap.add_argument("--quick", action="store_true", help="stages and raster band left to the built-in choice")
    ap.add_argument("--emit-table", metavar="PATH", help="write the winners of --out as the library's compiled-in table and exit")
    args = ap.parse_args(argv)
    if args.emit_table:
        print(f"{emit_table(args.out, args.emit_table)} entries written to {args.emit_table}")
        return 0
    shapes = [(n, n, n) for n in args.sizes] + [tuple(int(x) for x in t.lower().split("x")) for t in args.shapes]
    if any(len(t) != 3 or min(t) < 1 for t in shapes):
        ap.error("--shapes wants MxNxK with positive extents")
    probs = [Problem(m, n, k, l[0] == "T", l[1] == "T", args.dtype, args.with_c) for m, n, k in shapes for l in args.layouts]
    fn = (lambda p: candidates(p, tile_n=(64, 128, 256, 512), stages=(0,), raster_group=(0,))) if args.quick else candidates
    tune(probs, args.out, candidate_fn=fn)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
