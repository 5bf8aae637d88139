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


def test_loaded_tuning_entries_become_the_planner_choice(tmp_path):
    """gk_load_tuning: a measured entry replaces the planner's own choice for its problem and for
    problems close to it, explicit overrides still win, and clearing the table restores the planner."""
    import numpy as np
    import torch
    import gemmkernels_b200 as GK
    from gemmkernels_b200 import Layout, Operator, tuning as T
    from oracle import gemm_oracle as O

    def plan(m, n, k, **kw):
        conf = GK.get_config(gemm_shape=(m, n, k), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                             global_a_layout=Layout.ColMajor[GK.Float16], global_c_layout=Layout.Zero[GK.Float32],
                             global_d_layout=Layout.ColMajor[GK.Float32], **kw)
        a, b, d = GK.cuarray(GK.Float16, m, k), GK.cuarray(GK.Float16, k, n), GK.cuarray(GK.Float32, m, n)
        return conf, GK.query(conf, a, b, None, d)

    _, before = plan(2048, 2048, 2048)
    path = tmp_path / "r.jsonl"
    T.append_result(path, dict(problem="Float16:2048x2048x2048:NN", candidate="tn0-cg0-st0-rg0", tile_n=0, cta_group=0,
                               stages=0, raster_group=0, category="success", time_us=20.0))
    T.append_result(path, dict(problem="Float16:2048x2048x2048:NN", candidate="tn128-cg1-st3-rg0", tile_n=128, cta_group=1,
                               stages=3, raster_group=0, category="success", time_us=10.0))
    try:
        assert T.load_into_library(path) == 1
        _, p = plan(2048, 2048, 2048)
        assert (p.tile_n, p.cluster, p.stages) == (128, 1, 3)
        _, p = plan(2304, 1792, 2048)                       # within a factor 1.5 in every extent
        assert (p.tile_n, p.cluster) == (128, 1)
        _, p = plan(8192, 8192, 8192)                       # far away: the planner's own choice
        assert p.tile_n == 512
        _, p = plan(2048, 2048, 2048, tile_n=256, cta_group=2)     # an explicit override wins
        assert (p.tile_n, p.cluster) == (256, 2)
        # and the product computed with the loaded choice is still right
        rng = np.random.default_rng(2)
        A = rng.integers(-2, 3, (2048, 2048)).astype(np.float16); B = rng.integers(-2, 3, (2048, 2048)).astype(np.float16)
        conf, _ = plan(2048, 2048, 2048)
        d = GK.cuarray(GK.Float32, 2048, 2048)
        GK.matmul(conf, GK.to_cuarray(A), GK.to_cuarray(B), None, d)
        torch.cuda.synchronize(); GK.poll_status()
        assert np.array_equal(GK.to_numpy(d), O.gemm(A, B))
    finally:
        T.load_into_library(tmp_path / "empty.jsonl")       # no results: clears the table
    _, after = plan(2048, 2048, 2048)
    assert (after.tile_n, after.cluster, after.stages) == (before.tile_n, before.cluster, before.stages)
