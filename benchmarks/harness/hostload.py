"""Host load: a short measurement on the launch path is a CPU-contention measurement too.

A cell runs only on a quiet host, and the CPU that processes outside the cell's own tree burn while it runs is metered
in 0.5 s windows.  A window above ``LIMIT`` of the machine discards the attempt; a cell is retried at most ``ATTEMPTS``
times and a cell that never ran quiet is an error row.  The row records the windows' mean and maximum, the load
average and the discards.  Rule of the reference's meter (benchmarks/harness/host_load.py, benchmarks/README.md "Host
load").  Readings come from /proc/stat (machine) and /proc/<pid>/stat (the tree), both injectable for tests.
"""
from __future__ import annotations

import os
import threading
import time
from typing import Callable, Dict, List, Optional, Tuple

from .observer import proc_tree

WINDOW = 0.5
LIMIT = 0.10
ATTEMPTS = 3
_TICK = os.sysconf("SC_CLK_TCK") if hasattr(os, "sysconf") else 100


def machine_busy_ticks() -> Tuple[int, int]:
    """(user+nice+system ticks, cpu count) from /proc/stat."""
    with open("/proc/stat") as f:
        parts = f.readline().split()
    return int(parts[1]) + int(parts[2]) + int(parts[3]), os.cpu_count() or 1


def tree_ticks(root: int) -> int:
    tot = 0
    for pid in proc_tree(root):
        try:
            with open(f"/proc/{pid}/stat", "rb") as f:
                s = f.read().decode("latin-1")
            fields = s[s.rindex(")") + 2:].split()
            tot += int(fields[11]) + int(fields[12])
        except (OSError, ValueError, IndexError):
            continue
    return tot


class Meter:
    """Foreign CPU share per window: (machine busy - own tree) / (window * cpus)."""

    def __init__(self, root: Optional[int] = None, machine: Callable[[], Tuple[int, int]] = machine_busy_ticks,
                 tree: Optional[Callable[[], int]] = None, window: float = WINDOW, tick: int = _TICK):
        self.root = os.getpid() if root is None else root
        self.machine, self.tree = machine, tree or (lambda: tree_ticks(self.root))
        self.window, self.tick = window, tick
        self.windows: List[float] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def measure_window(self, seconds: Optional[float] = None, sleep=time.sleep) -> float:
        seconds = self.window if seconds is None else seconds
        m0, cpus = self.machine()
        t0 = self.tree()
        sleep(seconds)
        m1, _ = self.machine()
        t1 = self.tree()
        foreign = max(0, (m1 - m0) - (t1 - t0)) / self.tick
        share = foreign / (seconds * cpus)
        self.windows.append(share)
        return share

    def _run(self):
        while not self._stop.is_set():
            self.measure_window(sleep=lambda s: self._stop.wait(s))

    def __enter__(self):
        self.windows = []
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, name="bench-hostload", daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def summary(self) -> Dict[str, float]:
        w = self.windows or [0.0]
        try:
            load1 = os.getloadavg()[0]
        except OSError:
            load1 = None
        return {"windows": len(self.windows), "mean": sum(w) / len(w), "max": max(w), "loadavg_1m": load1}

    def quiet(self) -> bool:
        return max(self.windows or [0.0]) <= LIMIT


def wait_quiet(meter: Meter, windows: int = 4, tries: int = 20) -> bool:
    """True once ``windows`` consecutive windows were under the limit (checked before a sweep takes the device)."""
    run = 0
    for _ in range(tries * windows):
        run = run + 1 if meter.measure_window() <= LIMIT else 0
        if run >= windows:
            return True
    return False


def run_quiet(cell: Callable[[], dict], meter_factory: Callable[[], Meter] = Meter, attempts: int = ATTEMPTS) -> dict:
    """Run ``cell`` (returns a row) behind the meter: a loud attempt is discarded and rerun; the surviving row carries
    ``host_load``; no quiet attempt turns the row into an error row."""
    discards = []
    row: dict = {}
    for _ in range(attempts):
        meter = meter_factory()
        with meter:
            row = cell()
        s = meter.summary()
        if meter.quiet():
            row["host_load"] = {**s, "discards": discards}
            return row
        discards.append({"mean": s["mean"], "max": s["max"]})
    row = {k: v for k, v in row.items() if k not in ("requests",)}
    row.update(status="error", reason=f"the host was never quiet: {len(discards)} attempts each had a window above "
               f"{LIMIT:.0%} of the machine", host_load={"discards": discards})
    return row
