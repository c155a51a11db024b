"""Benchmark harness: result contract, request-window derivation, noise-aware verdicts, observer and host-load
bookkeeping, and the runner end to end on the host engine."""
import copy
import json
import random

import pytest

from benchmarks.harness import contract, hostload, runner, verdicts
from benchmarks.harness.observer import Observer, host_memory, proc_tree

SHA = "a" * 40


def make_row(tpot_ms=10.0, ttft_ms=50.0, osl=8, isl=128, **over):
    times = [1.0 + ttft_ms / 1e3 + i * tpot_ms / 1e3 for i in range(osl)]
    row = {"schema": 1, "framework": "poot_b200", "build_sha": SHA, "library_sha256": {"libpoot_kernels.so": "b" * 64},
           "nvcc_version": "12.9", "torch_version": "2.11", "model": "random:llama-3-8b", "scenario": "decode-curve",
           "isl": isl, "osl": osl, "synthetic_tokens": True, "prefix_cache": False, "placement": "single", "n_gpus": 1,
           "storage_dtype": "bf16", "compute_dtype": "bf16", "device": "NVIDIA B200", "driver_version": "580",
           "checkpoint_digest": "random:seed=0", "status": "ok",
           "requests": [{"prompt_tokens": isl, "start": 1.0, "token_times": times, "finish": times[-1] + 0.002,
                         "steps": osl}]}
    row.update(over)
    return row


def test_request_window_derivation_matches_the_definitions():
    row = make_row(tpot_ms=10.0, ttft_ms=50.0, osl=8)
    assert contract.row_errors(row) == []
    d = contract.derive_row(row)
    assert d["ttft_ms"] == pytest.approx(50.0) and d["tpot_ms"] == pytest.approx(10.0)
    assert d["decode_tok_s"] == pytest.approx(100.0) and d["finish_ms"] == pytest.approx(2.0)
    assert d["e2e_ms"] == pytest.approx(50.0 + 7 * 10.0 + 2.0)      # TTFT + sum(ITL) + finish
    assert d["itl_ms"]["n"] == 7 and "p99" not in d["itl_ms"]       # under 20 samples: median and range only
    long = contract.derive_row(make_row(osl=40))
    assert "p99" in long["itl_ms"]
    one = contract.derive_request({"start": 0.0, "token_times": [0.5], "finish": 0.6})
    assert one["tpot_ms"] is None and one["itl_ms"] == [] and one["ttft_ms"] == pytest.approx(500.0)
    zero = contract.derive_request({"start": 0.0, "token_times": [], "finish": 0.25})
    assert zero["ttft_ms"] is None and zero["finish_ms"] == pytest.approx(250.0) == zero["e2e_ms"]


def test_contract_refuses_rows_that_cannot_be_compared():
    def errs(mut):
        r = make_row()
        mut(r)
        return contract.row_errors(r)

    assert any("early stop" in e for e in errs(lambda r: r["requests"][0]["token_times"].pop()))
    assert any("outside its request" in e for e in errs(lambda r: r["requests"][0].update(steps=3)))
    assert any("not in order" in e for e in errs(lambda r: r["requests"][0].update(finish=0.5)))
    assert any("build_sha" in e for e in errs(lambda r: r.update(build_sha="deadbeef")))
    assert any("checkpoint_digest" in e for e in errs(lambda r: r.update(checkpoint_digest="md5:1")))
    assert any("disagrees" in e for e in errs(lambda r: r.update(decode_tok_s=123456.0)))
    assert any("unknown class" in e for e in errs(lambda r: r.update(memory_classes={"cache_bytes": 1})))
    assert any("states its reason" in e for e in errs(lambda r: r.update(status="refused")))
    refused = make_row(status="refused", reason="context longer than the model allows")
    del refused["requests"]
    assert contract.row_errors(refused) == []
    assert contract.row_errors([1, 2]) != []


def noisy(center, n, rel=0.004, seed=0, **kw):
    rng = random.Random(seed)
    return [make_row(tpot_ms=center * (1 + rng.uniform(-rel, rel)), ttft_ms=50.0 * (1 + rng.uniform(-rel, rel)), repeat=i, **kw)
            for i in range(n)]


def test_verdicts_follow_the_band_not_the_medians():
    pol = verdicts.load_policy()
    base = noisy(10.0, 5)
    same = verdicts.compare_sets(base, noisy(10.01, 5, seed=1), pol)
    assert [c["verdict"] for c in same] == [verdicts.WITHIN_NOISE] and verdicts.exit_code(same) == 0
    slow = verdicts.compare_sets(base, noisy(11.5, 5, seed=2), pol)
    assert slow[0]["verdict"] == verdicts.REGRESSION and verdicts.exit_code(slow) == 1
    fast = verdicts.compare_sets(base, noisy(8.0, 5, seed=3), pol)
    # the cell's verdict is the most serious of its metrics: a faster token with an unchanged first token is "within noise"
    assert fast[0]["entries"][0]["verdict"] == verdicts.IMPROVEMENT and fast[0]["verdict"] in verdicts.COMPARED
    assert verdicts.exit_code(fast) == 0
    few = verdicts.compare_sets(base[:3], noisy(10.0, 3, seed=4), pol)
    assert few[0]["verdict"] == verdicts.UNVERIFIED and "needs 5 runs" in few[0]["note"] and verdicts.exit_code(few) == 2
    wide = verdicts.compare_sets(noisy(10.0, 5, rel=0.2), noisy(10.2, 5, rel=0.2, seed=5), pol)
    assert wide[0]["verdict"] == verdicts.UNVERIFIED and "uncertainty" in wide[0]["note"]
    identical = verdicts.compare_sets([make_row() for _ in range(5)], [make_row() for _ in range(5)], pol)
    assert identical[0]["verdict"] == verdicts.UNVERIFIED and "identical" in identical[0]["note"]


def test_verdicts_for_broken_missing_and_mismatched_cells():
    pol = verdicts.load_policy()
    base = noisy(10.0, 5)
    failed = noisy(10.0, 4, seed=1) + [make_row(status="error", reason="device wait ran out")]
    assert verdicts.compare_sets(base, failed, pol)[0]["verdict"] == verdicts.REPEAT_FAILED
    dead = [make_row(status="error", reason="out of memory") for _ in range(5)]
    c = verdicts.compare_sets(base, dead, pol)[0]
    assert c["verdict"] == verdicts.CANDIDATE_FAILED and "out of memory" in c["note"]
    other = noisy(10.0, 5, seed=2, compute_dtype="fp8")
    assert verdicts.compare_sets(base, other, pol)[0]["verdict"] == verdicts.INCOMPARABLE
    mixed = noisy(10.0, 5, seed=3)
    mixed[2]["build_sha"] = "c" * 40
    assert verdicts.compare_sets(base, mixed, pol)[0]["verdict"] == verdicts.UNVERIFIED
    extra = noisy(10.0, 5, seed=4, isl=2048)
    cells = verdicts.compare_sets(base + extra, base, pol)
    assert sorted(c["verdict"] for c in cells) == sorted([verdicts.NOT_RUN, verdicts.WITHIN_NOISE])
    assert verdicts.exit_code(cells) == 2                   # a cell the baseline measured was not run: not a pass
    new = verdicts.compare_sets(base, noisy(10.0, 5, seed=6) + extra, pol)
    assert verdicts.NEW in [c["verdict"] for c in new] and verdicts.exit_code(new) == 0
    bad = copy.deepcopy(base)
    bad[0]["requests"][0]["steps"] = 1
    assert verdicts.compare_sets(bad, base, pol)[0]["verdict"] == verdicts.INVALID
    assert "| **regression** |" in verdicts.render(verdicts.compare_sets(base, noisy(12.0, 5, seed=9), pol))
    # a curve cell is judged at every metric: a good decode rate does not hide a slower first token
    slow_first = noisy(10.0, 5, seed=7)
    for r in slow_first:
        for q in r["requests"]:
            q["start"] -= 0.5
    c = verdicts.compare_sets(base, slow_first, pol)[0]
    assert c["verdict"] == verdicts.UNVERIFIED or c["verdict"] == verdicts.REGRESSION
    assert any(e["metric"] == "ttft_ms" and e["verdict"] in (verdicts.REGRESSION, verdicts.UNVERIFIED) for e in c["entries"])


def test_policy_file_is_checked():
    pol = verdicts.load_policy()
    assert pol["min_trials"] >= 2 and set(pol["metrics"]) >= {"decode_tok_s", "tpot_ms", "ttft_ms"}


def test_observer_keeps_peaks_per_phase():
    feed = iter([{"rss": 10, "vram": 100}, {"rss": 50, "vram": 900}, {"rss": 50, "vram": 900}, {"rss": 20, "vram": 400},
                 {"rss": 20, "vram": 400}, {"rss": 30, "vram": 500}, {"rss": 25, "vram": 450}])
    last = {}

    def host():
        nonlocal last
        last = next(feed, last)
        return {"rss": last["rss"]}

    t = [0.0]

    def clock():
        t[0] += 2.0
        return t[0]

    obs = Observer(root_pid=1, device_probe=lambda: {"vram": last["vram"]}, host_probe=host, clock=clock)
    obs.sample()                        # load: 10 / 100
    obs.sample()                        # load: 50 / 900  (the checkpoint staging peak)
    obs.mark("warmup")                  # samples on both sides of the boundary
    obs.mark("inference")
    obs.sample()
    obs.sample()
    r = obs.report()
    assert r["peak_vram_bytes"] == 900 and r["load_peak_vram_bytes"] == 900
    assert r["inference_peak_vram_bytes"] == 500 and r["inference_peak_rss_bytes"] == 30
    assert len(r["util_series"]) >= 5 and {s["phase"] for s in r["util_series"]} >= {"load", "inference"}
    with pytest.raises(ValueError):
        obs.mark("teardown")


def test_process_tree_memory_reads_this_process():
    import os
    assert os.getpid() in proc_tree(os.getpid())
    m = host_memory(os.getpid())
    assert m["rss"] > 0 and m["rss"] >= m["rss_anon"]


def test_host_load_meter_discards_loud_attempts():
    class FakeMeter(hostload.Meter):
        script = []

        def __init__(self):
            super().__init__(root=1, machine=lambda: (0, 4), tree=lambda: 0)
            self._w = FakeMeter.script.pop(0)

        def __enter__(self):
            self.windows = list(self._w)
            return self

        def __exit__(self, *exc):
            pass

    FakeMeter.script = [[0.02, 0.4], [0.01, 0.03]]
    row = hostload.run_quiet(lambda: make_row(), FakeMeter)
    assert row["status"] == "ok" and len(row["host_load"]["discards"]) == 1 and row["host_load"]["max"] == 0.03
    FakeMeter.script = [[0.5], [0.6], [0.7]]
    row = hostload.run_quiet(lambda: make_row(), FakeMeter)
    assert row["status"] == "error" and "never quiet" in row["reason"] and "requests" not in row
    # foreign share = (machine busy - own tree) / (window * cpus)
    ticks = iter([(0, 4), (200, 4)])
    own = iter([0, 100])
    m = hostload.Meter(root=1, machine=lambda: next(ticks), tree=lambda: next(own), tick=100)
    assert m.measure_window(0.5, sleep=lambda s: None) == pytest.approx(1.0 / (0.5 * 4))


def test_runner_end_to_end_on_the_host_engine(tmp_path):
    out = str(tmp_path / "run-r1")
    for rep in range(1, 3):
        row = runner.run_cell("fake", "decode-curve", 32, 16, repeat=rep, storage_dtype="f32")
        assert row["status"] == "ok", row.get("reason")
        assert contract.row_errors(row) == []
        assert len(row["requests"][0]["token_times"]) == 16 and row["requests"][0]["steps"] >= 16
        assert row["memory"]["peak_rss_bytes"] > 0 and row["checkpoint_digest"] == "random:seed=0"
        runner.append_row(out, row)
    rows = runner.load_rows(out)
    assert len(rows) == 2 and json.dumps(rows[0])
    from benchmarks.harness.__main__ import main
    assert main(["validate", out]) == 0
    assert main(["report", out]) == 0
    assert main(["compare", "--baseline", out, "--candidate", out]) == 2      # two repeats: unverified, never success
    refused = runner.run_cell("random:no-such-preset", "decode-curve", 8, 4)
    assert refused["status"] in ("refused", "error") and refused["reason"] and contract.row_errors(refused) == []
    with pytest.raises(FileNotFoundError):
        runner.load_rows(str(tmp_path / "nothing"))
