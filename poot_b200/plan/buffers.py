"""Buffer plan: lifetime colouring of intermediate values onto one arena
(crates/poot-graph-plan/src/buffer_plan.rs:1-7, src/entry_arena.rs:1-8).

Every value produced by a dispatching equation lives from its definition to its last use; values whose lifetimes do
not overlap may share bytes.  Views and aliases take no storage of their own; graph outputs and next-state values
stay live to the end of the step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

from ..ir.graph import Graph
from .planner import Plan

ALIGN = 256


@dataclass
class BufferPlan:
    offsets: Dict[int, Tuple[int, int]]      # value -> (offset, bytes)
    lifetimes: Dict[int, Tuple[int, int]]    # value -> (first eqn, last eqn)
    arena_bytes: int
    sum_bytes: int                           # what separate allocations would take


def first_fit(items, placed=None):
    """Place ``(key, size, start, end)`` intervals, in the order given, at the lowest offset no live interval holds.
    Returns ``({key: (offset, size)}, arena size, placed)``; ``placed`` (``[offset, size, start, end]`` lists) can be
    handed back in to continue a layout.  Shared by the value-level buffer plan and the launch program's arena."""
    placed = [] if placed is None else placed
    offsets = {}
    for key, size, s, t in items:
        busy = sorted((o, o + z) for o, z, a, b in placed if not (b < s or t < a))
        off = 0
        for lo, hi in busy:
            if off + size <= lo:
                break
            off = max(off, hi)
        placed.append([off, size, s, t])
        offsets[key] = (off, size)
    return offsets, max((o + z for o, z, _, _ in placed), default=0), placed


def plan_buffers(g: Graph, plans: List[Plan]) -> BufferPlan:
    last_use: Dict[int, int] = {}
    for k, e in enumerate(g.eqns):
        for v in e.inputs:
            last_use[v] = k
    end = len(g.eqns)
    for o in g.outputs:
        last_use[o.value] = end
    root: Dict[int, int] = {}                # view / alias outputs resolve to the value that owns the bytes
    for e, p in zip(g.eqns, plans):
        if p.kind in ("view", "alias"):
            root[e.outputs[0]] = root.get(e.inputs[0], e.inputs[0])
    for v, r in root.items():
        last_use[r] = max(last_use.get(r, 0), last_use.get(v, 0))
    life: Dict[int, Tuple[int, int]] = {}
    for k, (e, p) in enumerate(zip(g.eqns, plans)):
        if p.kind in ("view", "alias"):
            continue
        for v in e.outputs:
            life[v] = (k, last_use.get(v, k))
    # first-fit by decreasing size over the interval graph
    order = sorted(life, key=lambda v: (-g.types[v].nbytes, life[v][0]))
    items = [(v, (g.types[v].nbytes + ALIGN - 1) // ALIGN * ALIGN, life[v][0], life[v][1]) for v in order]
    offsets, arena, placed = first_fit(items)
    return BufferPlan(offsets, life, arena, sum(z for _, z, _, _ in placed))
