"""Target caps, timing snapshots, rooflines, weight roles."""
import json

import numpy as np
import pytest

from poot_b200 import target
from poot_b200.profile import ExecutionCounters, Report, TimingOptions, TimingSnapshot, decode_roofline, fused_collective_roofline
from poot_b200.utils import assert_close_scaled, run_contained, seeded_fill
from poot_b200.weights import WeightId, WeightMap, WeightRole, rank_view


def test_caps_read_measured_peaks(tmp_path):
    p = tmp_path / "peaks.json"
    p.write_text(json.dumps({"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1390.0}))
    c = target.b200(str(p))
    assert c.measured == "measured" and c.hbm_gbs == 6500.0 and c.bf16_tflops_sustained == 1390.0
    f = target.b200(str(tmp_path / "absent.json"))
    assert f.measured == "fallback" and f.hbm_gbs == 6650.0 and f.bf16_tflops == 1590.0
    assert c.sms == 148 and c.matrix.m == 128 and c.tma_x_multiple(2) == 8 and c.tma_x_multiple(4) == 4 and c.tma_x_multiple(1) == 16


def test_timing_snapshot_is_bounded_and_null_when_unmeasured():
    s = TimingSnapshot(TimingOptions("detailed", max_steps=3, max_dispatch_records=5))
    for i in range(5):
        s.record_step(64, 64, {"plan": 0.1, "launch": 0.2}, device_ms=5.0, spans=[("gemm", 100.0), ("attn", 40.0)])
    assert len(s.steps) == 3 and s.dropped_spans > 0
    r = Report.window(s, mark=2)
    assert len(r.steps) == 3 and r.device_ms() == 15.0 and abs(r.host_partitions()["launch"] - 0.6) < 1e-9
    c = TimingSnapshot()
    c.record_step(1, 1, {"plan": 0.1}, device_ms=3.0, spans=[("gemm", 1.0)])
    rep = Report.window(c)
    assert rep.device_ms() is None and rep.to_json()["device_ms"] is None and not rep.buckets()
    with pytest.raises(ValueError):
        TimingOptions("sometimes")
    k = ExecutionCounters()
    k.submit("compute", 3); k.wait("readback"); k.transfer(4096)
    assert k.submits["compute"] == 3 and k.waits["readback"] == 1 and k.transfer_bytes == 4096


def test_rooflines():
    caps = target.DeviceCaps(hbm_gbs=6500.0, bf16_tflops=1600.0, measured="measured")
    r = decode_roofline(16_000_000_000, 3.3, caps)
    assert r.bound == "hbm" and abs(r.achieved - 4848.5) < 1 and abs(r.fraction - 0.746) < 0.01 and "of measured" in str(r)
    # skinny o_proj at TP8: 64 x 4096 x 512, partial [64, 4096] bf16 to 7 peers, 4 MB of weights
    f = fused_collective_roofline(2 * 64 * 4096 * 512, 7 * 64 * 4096 * 2, 0.010, caps, hbm_bytes=4096 * 512 * 2)
    assert f.bound == "nvlink" and 0 < f.achieved < 1


def test_weight_ids_and_rank_views():
    wid = WeightId.parse("layers.3.experts.5.gate")
    assert wid == WeightId(WeightRole.MOE_GATE, 3, 5) and wid.canonical == "layers.3.experts.5.gate"
    assert WeightId.parse("embed").role is WeightRole.EMBED and WeightId.parse("layers.0.attn_q").layer == 0
    m = WeightMap({"embed": 1, "layers.0.attn_q": 2, "layers.0.bogus": 3})
    assert len(m) == 2 and m.unknown == ["layers.0.bogus"] and m[WeightId(WeightRole.ATTN_Q, 0)] == 2
    assert rank_view(WeightRole.ATTN_Q, (4096, 4096), 1, 8) == (slice(512, 1024), slice(None))
    assert rank_view(WeightRole.FFN_DOWN, (4096, 14336), 7, 8) == (slice(None), slice(12544, 14336))
    assert rank_view(WeightRole.ATTN_NORM, (4096,), 3, 8) == (slice(None),)
    with pytest.raises(ValueError):
        rank_view(WeightRole.FFN_GATE, (14336, 4096), 0, 5)
    from poot_b200.models.config import tiny_llama
    from poot_b200.models.model import Model
    names = {n: 0 for n in Model(tiny_llama()).weight_shapes()}
    assert WeightMap(names).missing(tiny_llama()) == []
    del names["layers.1.ffn_down"]
    assert WeightMap(names).missing(tiny_llama()) == [WeightId(WeightRole.FFN_DOWN, 1)]


def test_helpers():
    a = seeded_fill((4, 4), 1)
    assert np.array_equal(a, seeded_fill((4, 4), 1))
    assert_close_scaled(a + 1e-5, a, 1e-3)
    with pytest.raises(AssertionError):
        assert_close_scaled(a + 1.0, a, 1e-3)
    import sys
    r = run_contained([sys.executable, "-c", "import time; time.sleep(30)"], timeout=0.5)
    assert r.returncode == -9 and "deadline" in r.stderr
    assert run_contained([sys.executable, "-c", "print(7)"]).stdout.strip() == "7"


def test_flash_tiles_split_rules():
    import numpy as np
    from poot_b200.ops import cuda_ops as K
    seq = np.array([0] * 300 + [1] + [2] + [3] * 20 + [4] * 5)
    pos = np.concatenate([np.arange(300), [77], [12], np.arange(40, 60), np.arange(5)])
    tiles, covered = K.flash_tiles(seq, pos)
    assert tiles.tolist() == [[0, 128, 0, 0], [128, 128, 0, 128], [256, 44, 0, 256], [302, 20, 3, 40]]
    assert covered[:300].all() and not covered[300:302].any() and covered[302:322].all() and not covered[322:].any()
    # the same sequence at non-consecutive positions is two segments
    tiles, _ = K.flash_tiles(np.array([0] * 40), np.concatenate([np.arange(20), np.arange(100, 120)]))
    assert tiles.tolist() == [[0, 20, 0, 0], [20, 20, 0, 100]]
