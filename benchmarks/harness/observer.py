"""Memory and power are not self-reported: an observer thread samples them around the measured process.

Every ``interval`` seconds the observer reads total device memory in use and power (NVML through ``pynvml`` when it
loads, else one ``nvidia-smi --query-gpu`` call; reading only, no setting is touched) and the host memory of a process
tree (a ``/proc`` walk of the descendants: VmRSS split into RssAnon, the heap and staging buffers, and RssFile, a mapped
checkpoint and libraries).  It keeps the peaks per phase - the runner marks ``load`` -> ``warmup`` -> ``inference`` -
so a report can state the peak at inference (allocator, KV cache and kernels at steady state) beside the load peak,
and a 1 Hz trace.  Probes are plain callables, so tests drive the bookkeeping with fake ones.  Behaviour of the
reference's observer (benchmarks/harness/observer.py, benchmarks/harness/memory_phases.py).
"""
from __future__ import annotations

import os
import subprocess
import threading
import time
from typing import Callable, Dict, List, Optional

PHASES = ("load", "warmup", "inference")


def proc_tree(root: int) -> List[int]:
    """``root`` and its live descendants, from /proc/*/stat parent links."""
    parent: Dict[int, int] = {}
    for name in os.listdir("/proc"):
        if not name.isdigit():
            continue
        try:
            with open(f"/proc/{name}/stat", "rb") as f:
                s = f.read().decode("latin-1")
            parent[int(name)] = int(s[s.rindex(")") + 2:].split()[1])
        except (OSError, ValueError, IndexError):
            continue
    kids: Dict[int, List[int]] = {}
    for p, pp in parent.items():
        kids.setdefault(pp, []).append(p)
    out, todo = [], [root]
    while todo:
        p = todo.pop()
        out.append(p)
        todo += kids.get(p, [])
    return out


def host_memory(root: int) -> Dict[str, int]:
    """Bytes over the tree of ``root``: rss, rss_anon, rss_file."""
    tot = {"rss": 0, "rss_anon": 0, "rss_file": 0}
    for pid in proc_tree(root):
        try:
            with open(f"/proc/{pid}/status") as f:
                for line in f:
                    k, _, v = line.partition(":")
                    key = {"VmRSS": "rss", "RssAnon": "rss_anon", "RssFile": "rss_file"}.get(k)
                    if key:
                        tot[key] += int(v.split()[0]) * 1024
        except (OSError, ValueError):
            continue
    return tot


def nvml_probe() -> Optional[Callable[[], Dict[str, float]]]:
    """A callable that returns ``{"vram": bytes in use over all devices, "power": watts}``, or None without a device."""
    try:
        import pynvml
        pynvml.nvmlInit()
        hs = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in range(pynvml.nvmlDeviceGetCount())]
        if not hs:
            return None

        def read():
            return {"vram": float(sum(pynvml.nvmlDeviceGetMemoryInfo(h).used for h in hs)),
                    "power": sum(pynvml.nvmlDeviceGetPowerUsage(h) for h in hs) / 1000.0}
        read()
        return read
    except Exception:
        pass
    try:
        q = ["nvidia-smi", "--query-gpu=memory.used,power.draw", "--format=csv,noheader,nounits"]
        subprocess.run(q, check=True, capture_output=True, timeout=10)

        def read_smi():
            out = subprocess.run(q, check=True, capture_output=True, timeout=10, text=True).stdout
            rows = [[float(x) for x in line.split(",")] for line in out.strip().splitlines()]
            return {"vram": sum(r[0] for r in rows) * 2**20, "power": sum(r[1] for r in rows)}
        return read_smi
    except Exception:
        return None


class Observer:
    def __init__(self, root_pid: Optional[int] = None, interval: float = 0.25, device_probe="auto", host_probe=None,
                 clock=time.monotonic):
        self.root = os.getpid() if root_pid is None else root_pid
        self.interval = interval
        self.device_probe = nvml_probe() if device_probe == "auto" else device_probe
        self.host_probe = host_probe or (lambda: host_memory(self.root))
        self.clock = clock
        self.phase = PHASES[0]
        self.peaks: Dict[str, Dict[str, float]] = {}
        self.series: List[dict] = []
        self._last_series = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()

    def sample(self) -> dict:
        s = dict(self.host_probe())
        if self.device_probe is not None:
            try:
                s.update(self.device_probe())
            except Exception:
                pass
        now = self.clock()
        with self._lock:
            pk = self.peaks.setdefault(self.phase, {})
            for k, v in s.items():
                pk[k] = max(pk.get(k, 0), v)
            if self._last_series is None or now - self._last_series >= 1.0:
                self.series.append({"t": now, "phase": self.phase, **s})
                self._last_series = now
        return s

    def mark(self, phase: str) -> None:
        """Enter ``phase``; a sample is taken on both sides of the boundary so neither phase misses its edge."""
        if phase not in PHASES:
            raise ValueError(f"unknown phase {phase!r}")
        self.sample()
        with self._lock:
            self.phase = phase
        self.sample()

    def _run(self):
        while not self._stop.wait(self.interval):
            self.sample()

    def __enter__(self):
        self.sample()
        self._thread = threading.Thread(target=self._run, name="bench-observer", daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        self.sample()

    def report(self) -> dict:
        """Lifetime peaks (loading included), the peak at inference and the load peak, and the trace."""
        with self._lock:
            allp: Dict[str, float] = {}
            for pk in self.peaks.values():
                for k, v in pk.items():
                    allp[k] = max(allp.get(k, 0), v)
            inf, load = self.peaks.get("inference", {}), self.peaks.get("load", {})
            g = lambda d, k: int(d[k]) if k in d else None
            return {"peak_vram_bytes": g(allp, "vram"), "peak_rss_bytes": g(allp, "rss"),
                    "peak_rss_anon_bytes": g(allp, "rss_anon"), "peak_rss_file_bytes": g(allp, "rss_file"),
                    "inference_peak_vram_bytes": g(inf, "vram"), "inference_peak_rss_bytes": g(inf, "rss"),
                    "load_peak_vram_bytes": g(load, "vram"), "load_peak_rss_bytes": g(load, "rss"),
                    "peak_power_w": allp.get("power"), "util_series": list(self.series)}
