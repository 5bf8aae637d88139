"""Host logic of the benchmark runner (judgement, rendering, result files) and of the configuration
list, against the rules of benchmarks/runbenchmarks.jl:65-104, 221-300 and configs/configs.jl:492-690."""
import json

from gemmkernels_b200 import configs, runbenchmarks as R


def test_judge_uses_a_five_percent_band_on_the_ratio():
    assert R.judge(100.0, 100.0) == "invariant"
    assert R.judge(100.0, 104.9) == "invariant" and R.judge(100.0, 95.1) == "invariant"
    assert R.judge(100.0, 105.1) == "regression" and R.judge(100.0, 94.9) == "improvement"
    assert R.judge(100.0, float("nan")) == "regression"


def test_prettytime_and_prettyflops():
    times = [1500.0, 1600.0, 1550.0]                        # ns
    s = R.prettytime(times)
    assert s.startswith("1.55 μs ± ") and "(1.5 … 1.6 μs)" in s
    assert R.prettytime([2.0e6, 2.0e6]).startswith("2 ms ± 0%")
    assert R.prettyflops([1000.0, 500.0], {"M": 100, "N": 100, "K": 100}) == "4000 GFlops"   # 2e6 flop / 500 ns


def test_compare_reports_only_what_changed(tmp_path):
    before = {"a": {"times": [100.0, 110.0]}, "b": {"times": [100.0]}, "c `x`": {"times": [100.0]}, "gone": {"times": [1.0]}}
    after = {"a": {"times": [101.0, 99.0]}, "b": {"times": [120.0]}, "c `x`": {"times": [80.0, 90.0]}, "new": {"times": [1.0]}}
    det0 = {"a": {"grid": 148}, "b": {"grid": 148}, "c `x`": {"grid": 148}}
    det1 = {"a": {"grid": 128}, "b": {"grid": 148}, "c `x`": {"grid": 148}}
    j, report = R.compare(before, after, det0, det1, commit="abc", previous_commit="def")
    assert j == {"a": "invariant", "b": "regression", "c `x`": "improvement"}
    assert "comparing to def" in report
    rows = [l for l in report.splitlines() if l.startswith("| `")]
    assert len(rows) == 3                                   # a is listed because its launch details changed
    assert any(":x:" in r and "+20.0%" in r for r in rows) and any(":white_check_mark:" in r and "-20.0%" in r for r in rows)
    assert any("148 grid" in r and "128 grid" in r for r in rows)
    assert any(r.startswith("| ``c `x` `` |") for r in rows)   # names with backticks are fenced with longer runs
    _, quiet = R.compare(before, {"a": before["a"]})
    assert "No regressions or improvements detected." in quiet
    # files round-trip; reference-results.json wins over results.json
    R.save_results(tmp_path, after, det1)
    got = R.load_results(tmp_path)
    assert got["timings"] == after and got["details"] == det1
    (tmp_path / "reference-results.json").write_text(json.dumps(before))
    assert R.load_results(tmp_path)["timings"] == before
    assert R.load_results(tmp_path / "nowhere") is None


def test_configuration_list_matches_the_reference_families():
    cs = configs.get_configs()
    names = [c.name for c in cs]
    assert len(names) == len(set(names))
    count = lambda prefix: sum(n.startswith(prefix) for n in names)
    assert count("FPU GEMM") == 7 * 4 * 3 + 4 * 11 - 4     # 7 type triples x NN/NT/TN/TT x 3 sizes + op shapes (one shape shared)
    assert count("Tropical GEMM") == 16
    assert count("WMMA GEMM+bias") == 36 and count("WMMA diagonal GEMM") == 18
    assert count("WMMA Complex GEMM") == 36 and count("WMMA Dual GEMM") == 9
    assert "WMMA GEMM Float16*Float16+Float32=Float32 (2048×2048) · (2048×2048) (NN) Block (128, 128, 64) Warps (4, 2) OP (16, 16, 16)" in names
    assert "FPU GEMM Float32*Float32=Float64 (256×256) · (256×256) (TN) OP (8, 16, 2), base shape (4, 8, 1)" in names
    c = next(c for c in cs if c.name.startswith("WMMA GEMM+bias") and "(4096×4096)" in c.name)
    assert c.flops == 2.0 * 4096 ** 3 and c.shapes["bias"] == (4096,)
    quick = configs.get_configs(largest=False)
    assert all("2048" not in c.name and "4096" not in c.name for c in quick) and len(quick) < len(cs)
