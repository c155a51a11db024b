"""Multi-rank serving: rank 0 plans, every rank steps.

The driver, scheduler and HTTP server live on rank 0 only.  Before each device step rank 0 announces the
``StepInputs`` (a few KB of int32) and the block-table rows that changed; follower ranks replay the same step on
their shard so the in-kernel collectives meet (crates/poot-serve/src/batch/engine.rs:520-560 keeps one engine
thread per model for the same reason: one plan, many devices).

Announcements, readiness and acknowledgements go through the host control plane (``serve/control.py``), whose waits
are all bounded: rank 0 launches a step only after every follower said it is about to launch it too, so a follower that
left between two steps, or that stalls, is reported as ``RankLost`` before any kernel or collective could wait for it;
a follower that fails a step says so in its acknowledgement (``RankFailed``); a follower notices a dead rank 0 by its
heartbeat.  Whatever ends the group, rank 0 publishes the cause and the followers leave between two steps.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

from .control import ControlPlane, LeaderLost, RankFailed, RankLost  # noqa: F401  (re-exported)

_control: Optional[ControlPlane] = None


def init_control_group(rank: Optional[int] = None, world: Optional[int] = None, port: Optional[int] = None,
                       **limits) -> ControlPlane:
    """Connect this rank to the control plane (rank 0 hosts it).  Every rank calls it once at start-up.  The port
    defaults to ``POOT_CONTROL_PORT`` or the rendezvous port + 17."""
    global _control
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
    if port is None:
        port = int(os.environ.get("POOT_CONTROL_PORT", int(os.environ.get("MASTER_PORT", "29500")) + 17))
    _control = ControlPlane(rank, world, os.environ.get("MASTER_ADDR", "127.0.0.1"), port, **limits)
    _control.start_heartbeat()
    return _control


class LeaderStepEngine:
    """Wraps rank 0's step engine; mirrors block-table writes and step inputs to the followers."""

    def __init__(self, inner, control: Optional[ControlPlane] = None):
        self.inner = inner
        self.cp = control if control is not None else _control
        if self.cp is None:
            raise RuntimeError("init_control_group() must run before a LeaderStepEngine is built")
        self.max_tokens = inner.max_tokens
        self._tables: List[Tuple[int, list]] = []

    def __getattr__(self, name):            # timing fields, last_logits, copy_block ... of the wrapped engine
        return getattr(self.inner, name)

    def write_block_table(self, row: int, blocks) -> None:
        self._tables.append((row, list(blocks)))
        self.inner.write_block_table(row, blocks)

    def run_step(self, inp):
        n = self.cp.announce((self._tables, inp))
        self._tables = []
        try:
            self.cp.wait_ready(n)           # nothing is launched here unless every rank is about to launch too
            out = self.inner.run_step(inp)
            self.cp.wait_acks(n)
        except Exception as e:
            self.cp.stop(f"{type(e).__name__}: {e}")
            raise
        return out

    def abort(self) -> None:
        """Step-deadline watchdog hook: make pending device waits give up and tell the followers to stop."""
        self.cp.stop("step deadline exceeded on rank 0")
        if hasattr(self.inner, "abort"):
            self.inner.abort()

    def stop_followers(self, cause: str = "shutdown", linger: float = 5.0) -> None:
        self.cp.stop(cause, linger=linger)


def follow(engine, control: Optional[ControlPlane] = None, before_step=None) -> str:
    """Follower loop: replay every step rank 0 announces until it says stop; returns the cause of the stop and tells
    the control plane that this rank left.  ``before_step(n)`` is a test hook that runs between receiving step ``n`` and
    answering ready.  A control store that stops answering means rank 0 is gone: the loop ends between two steps."""
    cp = control if control is not None else _control
    cause = _follow(engine, cp, before_step)
    cp.leave(cause)
    return cause


def _follow(engine, cp: ControlPlane, before_step) -> str:
    while True:
        try:
            kind, payload = cp.next_step()
        except LeaderLost as e:
            return str(e)
        except Exception as e:          # the store went away with rank 0's process
            return f"rank 0 is gone ({type(e).__name__})"
        if kind == "stop":
            return payload
        n = cp.n - 1
        tables, inp = payload
        if before_step is not None:
            before_step(n)
        ended = cp.stopped()            # the group may have been ended while this rank was not looking
        if ended is not None:
            return ended
        try:
            cp.ready(n)
        except Exception as e:
            return f"rank 0 is gone ({type(e).__name__})"
        report = "ok"
        try:
            for row, blocks in tables:
                engine.write_block_table(row, blocks)
            engine.run_step(inp)
        except Exception as e:
            report = f"{type(e).__name__}: {e}"
        try:
            cp.ack(n, report)
        except Exception:
            pass
        if report != "ok":
            return f"this rank failed step {n}: {report}"
