"""The benchmark runner on the GPU: one configuration of every family of the list is timed (with its
cuBLAS baseline where it has one) and the result files compare clean against themselves."""
import pytest

pytestmark = pytest.mark.gpu


def test_runner_times_one_configuration_per_family(tmp_path):
    from gemmkernels_b200 import configs, runbenchmarks as R
    cs = configs.get_configs(largest=False)
    families = ["FPU GEMM Float16", "FPU GEMM Int32", "Tropical GEMM", "WMMA GEMM Float16*Float16+Float16", "WMMA GEMM Float16*Float16=Float32",
                "WMMA GEMM+bias", "WMMA diagonal GEMM", "WMMA Complex GEMM", "WMMA Dual GEMM"]
    picked = [next(c for c in cs if c.name.startswith(f)) for f in families]
    log = []
    results, baselines, details = R.run(picked, samples=5, log=log.append)
    assert set(results) == {c.name for c in picked}, log
    assert all(len(v["times"]) == 5 and all(1e2 < t < 1e9 for t in v["times"]) for v in results.values())
    assert all(details[k]["kernel"] in (1, 2, 3, 4) for k in results)
    assert any(k.startswith("WMMA GEMM Float16") for k in baselines) and not any(k.startswith("Tropical") for k in baselines)
    R.save_results(tmp_path, results, details)
    prev = R.load_results(tmp_path)
    judgements, report = R.compare(prev["timings"], results, prev["details"], details)
    assert set(judgements.values()) == {"invariant"} and "No regressions or improvements detected." in report
