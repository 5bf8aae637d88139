"""Host logic of the autotuner: sweep generation, resume from the results file, the timing loop and the
NVML helpers (against a fake NVML).  No GPU.  Reference behaviour mirrored: tuning/tune.jl:143-163
(measure until stable), :315-357 (checkpoint / resume), :223-247 (throttle wait)."""
import json

import pytest

from gemmkernels_b200 import tuning as T


def test_candidates_skip_refused_combinations():
    p = T.Problem(4096, 4096, 4096)
    cs = list(T.candidates(p))
    assert len(set(c.key() for c in cs)) == len(cs)
    assert all(not (c.cta_group == 2 and c.tile_n % 64) for c in cs)
    assert T.Candidate(256, 2, 0, 0, 1) in cs and T.Candidate(512, 2, 0, 0, 2) in cs
    assert not any(c.tile_n == 512 and c.cta_group == 1 for c in cs)
    assert cs[-1] == T.Candidate(0, 0, 0, 0)                # the built-in choice is measured too
    narrow = list(T.candidates(T.Problem(4096, 64, 4096)))
    assert narrow and all(c.tile_n in (0, 64) for c in narrow)


def test_resume_skips_measured_and_ignores_torn_lines(tmp_path):
    path = tmp_path / "r.jsonl"
    probs = [T.Problem(256, 256, 256), T.Problem(512, 512, 512, trans_b=True)]
    calls = []

    def fake(prob, cand):
        calls.append((prob.key(), cand.key()))
        if cand.tile_n == 192:
            return {"category": "config_error", "message": "refused"}
        if cand.stages == 3 and cand.cta_group == 2:
            raise RuntimeError("boom")
        return {"category": "success", "time_us": 100.0 + cand.tile_n / 8 - 10 * cand.cta_group + cand.stages}

    small = lambda p: T.candidates(p, raster_group=(0,))
    r1 = T.tune(probs[:1], path, measure=fake, candidate_fn=small, log=lambda s: None)
    n1 = len(calls)
    assert n1 == len(list(small(probs[0]))) == len(r1)
    # a run killed mid-write leaves a torn last line
    with open(path, "a") as f:
        f.write('{"problem": "Float16:512x512x512:NT", "candi')
    r2 = T.tune(probs, path, measure=fake, candidate_fn=small, log=lambda s: None)
    assert len(calls) - n1 == len(list(small(probs[1])))          # nothing of problem 0 re-measured
    assert all(k[0] != probs[0].key() for k in calls[n1:])
    cats = {r["category"] for r in r2.values()}
    assert cats == {"success", "config_error", "unknown_error"}
    b = T.best(r2, probs[0])
    assert b["cta_group"] == 2 and b["tile_n"] == 64 and b["stages"] == 0
    # every complete line of the file parses and carries its candidate's parameters
    lines = [l for l in path.read_text().splitlines() if l.endswith("}")]
    assert len(lines) == len(r2)
    assert all({"problem", "candidate", "tile_n", "category"} <= set(json.loads(l)) for l in lines)
    # a third run measures nothing
    n2 = len(calls)
    T.tune(probs, path, measure=fake, candidate_fn=small, log=lambda s: None)
    assert len(calls) == n2


def test_measure_until_stable_stops_after_patience():
    seq = iter([10.0, 9.0, 8.5, 8.5, 8.6, 8.49, 8.7, 1.0])
    n = [0]

    def run(batch):
        n[0] += 1
        return next(seq)

    assert T.measure_until_stable(run, patience=3) == pytest.approx(8.49)
    assert n[0] == 6                       # 8.49 is within the noise band: third stale batch


class FakeNvml:
    def __init__(self, masks):
        self.masks = list(masks)
        self.locked = None

    def nvmlDeviceGetCurrentClocksEventReasons(self, h):
        return self.masks.pop(0) if len(self.masks) > 1 else self.masks[0]

    def nvmlDeviceSetGpuLockedClocks(self, h, lo, hi):
        self.locked = (lo, hi)


def test_wait_if_throttled_polls_until_clear():
    slept = []
    nv = FakeNvml([0x40, 0x20, 0x4, 0x0])          # thermal, thermal, power cap only -> clear
    assert T.wait_if_throttled(nv, None, sleep=slept.append)
    assert len(slept) == 2
    nv = FakeNvml([0x8])
    assert not T.wait_if_throttled(nv, None, max_wait_s=1.0, poll_s=0.5, sleep=slept.append)


def test_lock_clocks_is_off_by_default():
    nv = FakeNvml([0])
    with pytest.raises(PermissionError):
        T.lock_clocks(nv, None, 1500)
    assert nv.locked is None
    T.lock_clocks(nv, None, 1500, i_understand_this_outlasts_the_process=True)
    assert nv.locked == (1500, 1500)


def test_winners_and_emitted_table(tmp_path):
    """The sweep's winners become the library's defaults: one entry per problem whose best candidate
    beats the planner's own choice by 2 % or more, written as the initialiser list the library compiles in."""
    path = tmp_path / "r.jsonl"
    def rec(pk, tn, cg, st, rg, t, cat="success", kps=0):
        T.append_result(path, dict(problem=pk, candidate=T.Candidate(tn, cg, st, rg, kps).key(), tile_n=tn, cta_group=cg,
                                   stages=st, raster_group=rg, k_blocks_per_stage=kps, category=cat, time_us=t))
    rec("Float16:2048x2048x2048:NN", 0, 0, 0, 0, 20.9)
    rec("Float16:2048x2048x2048:NN", 256, 1, 4, 0, 19.0, kps=2)   # 10 % faster than the planner: an entry
    rec("Float16:2048x2048x2048:NN", 128, 2, 0, 0, 5.0, cat="invalid_result")   # fast but wrong: never a winner
    rec("TF32:4096x4096x4096:TN+C", 0, 0, 0, 0, 100.0)
    rec("TF32:4096x4096x4096:TN+C", 256, 2, 0, 8, 99.5)           # within the margin: no entry
    rec("BFloat16:8192x1024x8192:NT", 512, 2, 0, 0, 80.0)         # planner not measured: the best stands
    w = T.winners(T.load_results(path))
    assert [e["problem"] for e in w] == ["BFloat16:8192x1024x8192:NT", "Float16:2048x2048x2048:NN"]
    assert w[1] == dict(w[1], dtype=0, trans_a=0, trans_b=0, has_c=0, m=2048, n=2048, k=2048, tile_n=256, cta_group=1,
                        stages=4, raster_group=0, k_blocks_per_stage=2)
    assert w[0]["dtype"] == 1 and w[0]["trans_b"] == 1 and (w[0]["m"], w[0]["n"], w[0]["k"]) == (8192, 1024, 8192)
    out = tmp_path / "tuned_table.inc"
    assert T.emit_table(path, out) == 2
    text = out.read_text()
    assert "{0, 0, 0, 0, 2048, 2048, 2048, 256, 1, 4, 0, 2, 0}," in text and "{1, 0, 1, 0, 8192, 1024, 8192, 512, 2, 0, 0, 0, 0}," in text
    assert all(l.startswith("//") or l.startswith("    {") for l in text.splitlines())


def test_compiled_in_table_is_well_formed():
    """csrc/tuned_table.inc is generated: comment lines and 11-field initialisers only."""
    from pathlib import Path
    import re
    inc = Path(T.__file__).resolve().parents[1] / "csrc" / "tuned_table.inc"
    for line in inc.read_text().splitlines():
        if line.strip() and not line.lstrip().startswith("//"):
            m = re.match(r"\s*\{([^}]*)\},", line)
            assert m and len(m.group(1).split(",")) == 13, line
