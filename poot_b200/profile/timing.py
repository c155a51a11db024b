"""Always-on counters and an opt-in, bounded record of per-step and per-launch device time.

``TimingOptions`` is typed configuration (never an environment variable): ``counters_only`` keeps the cumulative
``ExecutionCounters``; ``detailed`` additionally brackets launches with CUDA events (eager steps) or each graph replay
(captured steps) and folds the spans into a ``TimingSnapshot`` bounded by ``max_steps`` / ``max_dispatch_records``.
A time that was not measured is ``None``, never 0 (website/docs/serve/configuration.md:74-86).
"""
from __future__ import annotations

from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TimingOptions:
    mode: str = "counters_only"          # counters_only | detailed
    max_steps: int = 4096
    max_dispatch_records: int = 65536
    sample_every: int = 1

    def __post_init__(self):
        if self.mode not in ("counters_only", "detailed"):
            raise ValueError(f"timing mode {self.mode!r}")
        if self.max_steps < 1 or self.max_dispatch_records < 1 or self.sample_every < 1:
            raise ValueError("timing bounds must be positive")


PURPOSES = ("compute", "upload", "readback", "validation", "timing")


@dataclass
class ExecutionCounters:
    """Logical launches and replays, physical submits and waits by purpose, transfer ops and bytes
    (crates/poot-runtime-common/src/telemetry.rs:12-80)."""
    dispatches: int = 0
    replays: int = 0
    submits: Dict[str, int] = field(default_factory=lambda: {p: 0 for p in PURPOSES})
    waits: Dict[str, int] = field(default_factory=lambda: {p: 0 for p in PURPOSES})
    transfer_ops: int = 0
    transfer_bytes: int = 0

    def submit(self, purpose: str, n: int = 1) -> None:
        self.submits[purpose] += n

    def wait(self, purpose: str, n: int = 1) -> None:
        self.waits[purpose] += n

    def transfer(self, nbytes: int) -> None:
        self.transfer_ops += 1
        self.transfer_bytes += int(nbytes)


@dataclass
class StepRecord:
    index: int
    tokens: int
    rows: int
    host_ms: Dict[str, float]                     # partitions: plan, upload, launch, readback
    device_ms: Optional[float] = None             # None = not measured
    spans: List[Tuple[str, float]] = field(default_factory=list)     # (kernel, microseconds)


class TimingSnapshot:
    def __init__(self, options: Optional[TimingOptions] = None):
        self.options = options or TimingOptions()
        self.steps: Deque[StepRecord] = deque(maxlen=self.options.max_steps)
        self.counters = ExecutionCounters()
        self._records = 0
        self._seen = 0
        self.dropped_spans = 0

    @property
    def detailed(self) -> bool:
        return self.options.mode == "detailed"

    def record_step(self, tokens: int, rows: int, host_ms: Dict[str, float], device_ms: Optional[float] = None,
                    spans: Optional[List[Tuple[str, float]]] = None) -> None:
        self._seen += 1
        if self._seen % self.options.sample_every:
            return
        spans = list(spans or []) if self.detailed else []
        room = self.options.max_dispatch_records - self._records
        if len(spans) > room:
            self.dropped_spans += len(spans) - max(room, 0)
            spans = spans[:max(room, 0)]
        self._records += len(spans)
        if len(self.steps) == self.steps.maxlen and self.steps:
            self._records -= len(self.steps[0].spans)
        self.steps.append(StepRecord(self._seen, tokens, rows, dict(host_ms), device_ms if self.detailed else None, spans))

    def mark(self) -> int:
        return self._seen


class Report:
    """A window of a snapshot rendered as op buckets and host partitions."""

    def __init__(self, steps: List[StepRecord]):
        self.steps = steps

    @staticmethod
    def window(snapshot: TimingSnapshot, mark: int = 0, entries: Optional[int] = None) -> "Report":
        steps = [s for s in snapshot.steps if s.index > mark]
        return Report(steps[-entries:] if entries else steps)

    def buckets(self) -> "OrderedDict[str, Tuple[int, float]]":
        agg: Dict[str, List[float]] = {}
        for s in self.steps:
            for name, us in s.spans:
                a = agg.setdefault(name, [0, 0.0])
                a[0] += 1
                a[1] += us
        return OrderedDict(sorted(((k, (int(c), t)) for k, (c, t) in agg.items()), key=lambda kv: -kv[1][1]))

    def host_partitions(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        for s in self.steps:
            for k, v in s.host_ms.items():
                out[k] = out.get(k, 0.0) + v
        return out

    def device_ms(self) -> Optional[float]:
        vals = [s.device_ms for s in self.steps if s.device_ms is not None]
        return sum(vals) if vals else None

    def to_json(self) -> dict:
        return {"steps": len(self.steps), "device_ms": self.device_ms(), "host_ms": self.host_partitions(),
                "buckets": {k: {"count": c, "us": t} for k, (c, t) in self.buckets().items()}}

    def render(self) -> str:
        b = self.buckets()
        total = sum(t for _, t in b.values()) or 1.0
        lines = [f"{len(self.steps)} steps, device {self.device_ms()} ms"]
        for k, (c, t) in b.items():
            lines.append(f"  {t:10.1f} us {100 * t / total:5.1f}%  x{c:<5d} {k}")
        return "\n".join(lines)
