"""Serving metrics: counters, gauges and fixed-bucket histograms rendered as JSON and Prometheus text.

Names follow the reference (website/docs/architecture/serving-design.mdx:65-76; crates/poot-serve/src/metrics.rs:
20-365): ``poot_ttft_ms``, ``poot_itl_ms``, ``poot_request_e2e_ms``, ``poot_queue_wait_ms`` histograms; request /
token counters; prefix-cache hit and query tokens; in-flight, queue depth, batch size, KV usage gauges.  Every
value is produced by the engine itself, never read from a vendor tool.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List

BUCKETS_MS = [1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 30000, 60000]


class Histogram:
    def __init__(self):
        self.counts = [0] * (len(BUCKETS_MS) + 1)
        self.sum, self.n = 0.0, 0

    def observe(self, v: float) -> None:
        self.sum += v
        self.n += 1
        for i, b in enumerate(BUCKETS_MS):
            if v <= b:
                self.counts[i] += 1
                return
        self.counts[-1] += 1

    def quantile(self, q: float) -> float:
        if self.n == 0:
            return 0.0
        target, acc = q * self.n, 0
        for i, c in enumerate(self.counts):
            acc += c
            if acc >= target:
                return float(BUCKETS_MS[i]) if i < len(BUCKETS_MS) else float("inf")
        return float("inf")


class Metrics:
    HISTS = ("poot_ttft_ms", "poot_itl_ms", "poot_request_e2e_ms", "poot_queue_wait_ms")
    COUNTERS = ("poot_requests_total", "poot_requests_completed_total", "poot_requests_cancelled_total",
                "poot_requests_errored_total", "poot_requests_rejected_total", "poot_prompt_tokens_total",
                "poot_completion_tokens_total", "poot_prefix_cache_hit_tokens_total",
                "poot_prefix_cache_query_tokens_total", "poot_engine_steps_total", "poot_engine_compiles_total",
                "poot_step_deadline_exceeded_total")
    GAUGES = ("poot_inflight_requests", "poot_queue_depth", "poot_batch_size", "poot_slot_capacity",
              "poot_kv_usage_ratio", "poot_kv_blocks_used", "poot_kv_blocks_total", "poot_prefix_hit_rate",
              "poot_gpu_active_ratio", "poot_weight_bytes", "poot_kv_bytes", "poot_uptime_seconds")

    def __init__(self):
        self.lock = threading.Lock()
        self.h: Dict[str, Histogram] = {n: Histogram() for n in self.HISTS}
        self.c: Dict[str, float] = {n: 0 for n in self.COUNTERS}
        self.g: Dict[str, float] = {n: 0 for n in self.GAUGES}
        self.started = time.time()

    def inc(self, name: str, v: float = 1) -> None:
        with self.lock:
            self.c[name] += v

    def set(self, name: str, v: float) -> None:
        with self.lock:
            self.g[name] = v

    def observe(self, name: str, v: float) -> None:
        with self.lock:
            self.h[name].observe(v)

    def to_json(self) -> dict:
        with self.lock:
            self.g["poot_uptime_seconds"] = time.time() - self.started
            q = self.c["poot_prefix_cache_query_tokens_total"]
            self.g["poot_prefix_hit_rate"] = self.c["poot_prefix_cache_hit_tokens_total"] / q if q else 0.0
            out = {"counters": dict(self.c), "gauges": dict(self.g), "histograms": {}}
            for n, h in self.h.items():
                out["histograms"][n] = {"count": h.n, "sum": h.sum, "p50": h.quantile(0.5), "p95": h.quantile(0.95),
                                        "p99": h.quantile(0.99), "buckets": dict(zip(map(str, BUCKETS_MS + ["+Inf"]), h.counts))}
            return out

    def to_prometheus(self) -> str:
        j = self.to_json()
        lines: List[str] = []
        for n, v in j["counters"].items():
            lines += [f"# TYPE {n} counter", f"{n} {v}"]
        for n, v in j["gauges"].items():
            lines += [f"# TYPE {n} gauge", f"{n} {v}"]
        for n, h in self.h.items():
            lines.append(f"# TYPE {n} histogram")
            acc = 0
            for b, c in zip(BUCKETS_MS + ["+Inf"], h.counts):
                acc += c
                lines.append(f'{n}_bucket{{le="{b}"}} {acc}')
            lines += [f"{n}_sum {h.sum}", f"{n}_count {h.n}"]
        return "\n".join(lines) + "\n"
