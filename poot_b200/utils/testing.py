"""Test helpers used across the suite."""
from __future__ import annotations

import subprocess
import sys
from typing import Optional, Sequence

import numpy as np


def seeded_fill(shape, seed: int, std: float = 1.0, dtype=np.float32) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal(shape) * std).astype(dtype)


def assert_close_scaled(got, want, rel: float = 1e-3, what: str = "") -> None:
    """Max abs error relative to the reference's own scale (a bf16 result is judged against max|want|, not per element)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    if got.shape != want.shape:
        raise AssertionError(f"{what}: shape {got.shape} vs {want.shape}")
    scale = max(1.0, float(np.abs(want).max()) if want.size else 1.0)
    err = float(np.abs(got - want).max()) / scale if want.size else 0.0
    if not np.isfinite(got).all() or err > rel:
        raise AssertionError(f"{what}: scaled error {err:.3e} > {rel:.1e}")


def run_contained(argv: Sequence[str], timeout: float = 120.0, env: Optional[dict] = None) -> subprocess.CompletedProcess:
    """Run a child in its own session with a deadline; on expiry only that child's process group is ended
    (crates/poot-test-util/src/contained_child.rs:1-9)."""
    import os
    import signal
    p = subprocess.Popen(list(argv), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True, env=env)
    try:
        out, err = p.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGKILL)
        out, err = p.communicate()
        return subprocess.CompletedProcess(argv, -9, out, err + "\n[deadline expired]")
    return subprocess.CompletedProcess(argv, p.returncode, out, err)
