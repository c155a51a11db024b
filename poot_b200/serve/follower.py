"""Multi-rank serving: rank 0 plans, every rank steps.

The driver, scheduler and HTTP server live on rank 0 only.  Before each device step rank 0 broadcasts the
``StepInputs`` (a few KB of int32) and the block-table rows that changed; follower ranks replay the same step on
their shard so the in-kernel collectives meet (crates/poot-serve/src/batch/engine.rs:520-560 keeps one engine
thread per model for the same reason: one plan, many devices).
"""
from __future__ import annotations

import pickle
from typing import List, Tuple

import numpy as np


_control = None


def init_control_group():
    """A host-side (gloo) group for the step announcements, so they never touch the GPU streams.  Collective: every
    rank calls it once after ``init_process_group``."""
    global _control
    import torch.distributed as dist
    _control = dist.new_group(backend="gloo")
    return _control


def _bcast_obj(obj, src: int = 0):
    import torch.distributed as dist
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=_control)
    return box[0]


class LeaderStepEngine:
    """Wraps rank 0's step engine; mirrors block-table writes and step inputs to the followers."""

    def __init__(self, inner):
        self.inner = inner
        self.max_tokens = inner.max_tokens
        self._tables: List[Tuple[int, list]] = []

    def write_block_table(self, row: int, blocks) -> None:
        self._tables.append((row, list(blocks)))
        self.inner.write_block_table(row, blocks)

    def run_step(self, inp):
        _bcast_obj(("step", self._tables, inp))
        self._tables = []
        return self.inner.run_step(inp)

    def stop_followers(self) -> None:
        _bcast_obj(("stop", None, None))


def follow(engine) -> None:
    """Follower loop: replay every step rank 0 announces until it says stop."""
    while True:
        kind, tables, inp = _bcast_obj(None)
        if kind == "stop":
            return
        for row, blocks in tables:
            engine.write_block_table(row, blocks)
        engine.run_step(inp)
