"""The autotuner's GPU leg on a small problem: every candidate is verified against the built-in
configuration's output, timed with CUDA events, and the results file resumes."""
import pytest

pytestmark = pytest.mark.gpu


def test_quick_sweep_512(tmp_path):
    from gemmkernels_b200 import tuning as T
    prob = T.Problem(512, 512, 512, trans_b=True)
    path = tmp_path / "t.jsonl"
    fn = lambda p: T.candidates(p, stages=(0, 3), raster_group=(0,))
    res = T.tune([prob], path, candidate_fn=fn, log=lambda s: None)
    cats = [r["category"] for r in res.values()]
    assert cats.count("success") >= 6, cats
    assert set(cats) <= {"success", "config_error"}, res          # nothing wrong, nothing timed out
    ok = [r for r in res.values() if r["category"] == "success"]
    assert all(r["rel_error"] <= 1e-3 and 1.0 < r["time_us"] < 1e4 for r in ok)
    assert T.best(res, prob)["time_us"] == min(r["time_us"] for r in ok)
    # resume: nothing is measured twice
    calls = []
    T.tune([prob], path, measure=lambda p, c: calls.append(c) or {"category": "success", "time_us": 1.0},
           candidate_fn=fn, log=lambda s: None)
    assert calls == []
