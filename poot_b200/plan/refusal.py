"""Typed refusals: what the planner could not place, and why (crates/poot-graph-plan/src/refusal.rs:1-4)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass
class Refusal(Exception):
    eqn: int
    op: str
    dtypes: Tuple[str, ...]
    target: str
    missing: str

    def __str__(self) -> str:
        return f"eqn {self.eqn} ({self.op} over {', '.join(self.dtypes)}) has no kernel on {self.target}: {self.missing}"
