"""Benchmark / regression runner over the configuration list — what benchmarks/runbenchmarks.jl does
for the reference: time every configuration (and its cuBLAS baseline), write `results.json` and
`details.json`, and judge the minima against a previous run with a ±5 % tolerance
(runbenchmarks.jl:229-243), printing the reference's markdown table for what changed.

    python -m gemmkernels_b200.runbenchmarks [--filter TEXT] [--samples N] [--out DIR] [--previous DIR]

Times are per-launch device times in nanoseconds (CUDA events between back-to-back launches); the
reference takes them from the CUDA profiler (runbenchmarks.jl:124-141).  `details` holds what
`gk_gemm_query` reports for the launch (kernel family, grid, shared memory, TMEM columns) where the
reference recorded registers and shared memory.  The CI-bot parts (cloning the results branch, posting
a GitHub comment, runbenchmarks.jl:12-24, 340-end) are not reproduced.
"""
from __future__ import annotations

import json
import math
import statistics
from pathlib import Path

NUM_SAMPLES = 200
TOLERANCE = 0.05


# ---------------------------------------------------------------------------------------------------
# rendering (runbenchmarks.jl:65-104)
# ---------------------------------------------------------------------------------------------------
def _sig(x: float, digits: int) -> float:
    if x == 0 or not math.isfinite(x):
        return x
    return round(x, digits - 1 - int(math.floor(math.log10(abs(x)))))


def prettyflops(times_ns, matmul_shape) -> str:
    t = min(times_ns)
    m, n, k = (matmul_shape[c] for c in "MNK")
    return f"{_sig(2.0 * m * n * k / t, 4):g} GFlops"


def prettytime(times_ns) -> str:
    t = statistics.fmean(times_ns)
    sigma = statistics.stdev(times_ns) if len(times_ns) > 1 else 0.0
    lo, hi = min(times_ns), max(times_ns)
    scale, unit = (1, "ns") if t < 1e3 else (1e3, "μs") if t < 1e6 else (1e6, "ms") if t < 1e9 else (1e9, "s")
    cv = _sig(100 * sigma / abs(t), 3) if t else 0.0
    return f"{_sig(t / scale, 3):g} {unit} ± {cv:g}% ({_sig(lo / scale, 3):g} … {_sig(hi / scale, 3):g} {unit})"


# ---------------------------------------------------------------------------------------------------
# judgement (runbenchmarks.jl:221-248)
# ---------------------------------------------------------------------------------------------------
def judge(old: float, new: float, tolerance: float = TOLERANCE) -> str:
    r = new / old if old else float("nan")
    if math.isnan(r) or (r - tolerance) > 1.0:
        return "regression"
    if (r + tolerance) < 1.0:
        return "improvement"
    return "invariant"


def _code(s: str) -> str:
    runs = [len(m) for m in __import__("re").findall(r"`+", s)]
    if not runs:
        return f"`{s}`"
    ticks = "`" * (max(runs) + 1)
    return f"{ticks}{' ' if s.startswith('`') else ''}{s}{' ' if s.endswith('`') else ''}{ticks}"


def compare(before: dict, after: dict, before_details: dict | None = None, after_details: dict | None = None,
            commit: str = "HEAD", previous_commit: str = "local") -> tuple[dict, str]:
    """-> ({name: judgement} for the names both runs have, markdown report of what changed)."""
    bmin = {k: min(v["times"]) for k, v in before.items()}
    amin = {k: min(v["times"]) for k, v in after.items()}
    judgements = {k: judge(bmin[k], amin[k]) for k in bmin.keys() & amin.keys()}
    lines = [f"Benchmark results for commit {commit} (comparing to {previous_commit}):"]

    def details_changed(k):
        if not before_details or not after_details or k not in before_details or k not in after_details:
            return False
        return before_details[k] != after_details[k]

    shown = {k: v for k, v in judgements.items() if v != "invariant" or details_changed(k)}
    if not shown:
        lines.append("No regressions or improvements detected.")
    else:
        lines += ["", "| test | master | PR | Δmin |", "|------|--------|----|------|"]
        for k in sorted(shown):
            old, new = prettytime(before[k]["times"]), prettytime(after[k]["times"])
            if details_changed(k):
                for key in sorted(set(before_details[k]) | set(after_details[k])):
                    if before_details[k].get(key) != after_details[k].get(key):
                        old += f"<br>{before_details[k].get(key)} {key}"
                        new += f"<br>{after_details[k].get(key)} {key}"
            mark = {"regression": ":x:", "improvement": ":white_check_mark:"}.get(shown[k], "")
            lines.append(f"| {_code(k)} | {old} | {new} | {100 * (amin[k] / bmin[k] - 1):+.1f}% {mark} |")
    return judgements, "\n".join(lines)


def load_results(directory) -> dict | None:
    """Previous `results.json` (+ `details.json`) of a directory, or None (runbenchmarks.jl:27-56)."""
    d = Path(directory)
    rf = next((p for p in (d / "reference-results.json", d / "results.json") if p.is_file()), None)
    if rf is None:
        return None
    df = rf.with_name(rf.name.replace("results", "details"))
    return {"commit": "local", "timings": json.loads(rf.read_text()),
            "details": json.loads(df.read_text()) if df.is_file() else None}


def save_results(directory, results: dict, details: dict) -> None:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    (d / "results.json").write_text(json.dumps(results))
    (d / "details.json").write_text(json.dumps(details))


# ---------------------------------------------------------------------------------------------------
# measurement
# ---------------------------------------------------------------------------------------------------
def time_launches(launch, samples: int) -> list:
    """Device time of each of `samples` back-to-back launches, in ns."""
    import torch
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(samples + 1)]
    ev[0].record()
    for i in range(samples):
        launch()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return [ev[i].elapsed_time(ev[i + 1]) * 1e6 for i in range(samples)]


def run(configs, samples: int = NUM_SAMPLES, log=print) -> tuple[dict, dict, dict]:
    """-> (results, baseline_results, details), keyed by configuration name."""
    import torch
    from .config import ConfigError
    from .matmul import poll_status, query
    results, baselines, details = {}, {}, {}
    for idx, cf in enumerate(configs):
        log(f"Running benchmark {idx + 1}/{len(configs)} {cf.name}...")
        try:
            ops = cf.generate_inputs(idx)
            launch = cf.bind(ops)
            launch()                                    # warm-up
            torch.cuda.synchronize()
            times = time_launches(launch, samples)
            poll_status()
            plan = query(cf.config, ops["a"], ops["b"], ops.get("c"), ops["d"], kernel=cf.kernel, **cf.kwargs(ops))
            details[cf.name] = {"kernel": int(plan.kernel), "grid": int(plan.grid), "dynamic_shared_mem": int(plan.smem_bytes),
                                "tmem_columns": int(plan.tmem_columns), "tile": [int(plan.tile_m), int(plan.tile_n), int(plan.tile_k)]}
            log(f"\tGemmKernels: {prettytime(times)} {prettyflops(times, cf.config.matmul_shape)}")
            if cf.baseline is not None:
                cf.baseline(ops)
                torch.cuda.synchronize()
                btimes = time_launches(lambda: cf.baseline(ops), samples)
                log(f"\tBaseline:    {prettytime(btimes)} {prettyflops(btimes, cf.config.matmul_shape)} "
                    f"(GemmKernels: {_sig(100 * min(btimes) / min(times), 3):g}%)")
                baselines[cf.name] = {"times": btimes}
            results[cf.name] = {"times": times}
        except ConfigError as err:
            log(f"Skipping benchmark {cf.name}: Invalid configuration: {err}.")
    return results, baselines, details


def main(argv=None) -> int:
    import argparse
    from .configs import get_configs
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--filter", default="", help="only configurations whose name contains this text")
    ap.add_argument("--samples", type=int, default=NUM_SAMPLES)
    ap.add_argument("--out", default=".", help="directory for results.json and details.json")
    ap.add_argument("--previous", default=None, help="directory holding the run to compare with (default: --out)")
    ap.add_argument("--quick", action="store_true", help="leave out the 2048 / 4096 cases")
    args = ap.parse_args(argv)
    previous = load_results(args.previous or args.out)
    print("No previous benchmark results found" if previous is None else f"Found previous timings for commit {previous['commit']}")
    cfs = [c for c in get_configs(largest=not args.quick) if args.filter in c.name]
    results, baselines, details = run(cfs, args.samples)
    save_results(args.out, results, details)
    if baselines:
        (Path(args.out) / "baseline-results.json").write_text(json.dumps(baselines))
    if previous is not None:
        judgements, report = compare(previous["timings"], results, previous["details"], details)
        print("Improvements:", *[k for k, v in judgements.items() if v == "improvement"], sep="\n")
        print("Regressions:", *[k for k, v in judgements.items() if v == "regression"], sep="\n")
        print(report)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
