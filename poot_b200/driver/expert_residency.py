"""Expert residency: which experts of each routed layer sit in which rows of a device-resident pool.

A routed model whose expert tables do not fit the device (DeepSeek-V3 in bf16 is 1.3 TB of experts; one B200 has 180 GB)
keeps every expert in pinned host memory and only ``P < E`` of them per layer in a device pool ``[P, ...]``.  A step's
routed layer is cut at the router: the host reads the step's expert ids, this manager pins the experts the step needs,
picks rows for the misses - free rows first, then the least recently used row that no needed expert holds - and answers
with the rows to refill and the ``[E]`` map from expert id to pool row (``-1`` = not resident).  The engine copies the
stored bytes of each named expert into its row and runs the layer over the pool through the map; the manager never
holds weight bytes.  One LRU per site (a layer's up and down tables share a site, so both get the same expert in the
same row).

Behaviour of the reference's manager and pool transform (crates/poot-llm/src/driver/expert_residency.rs:1-14,
crates/poot-graph-plan/src/passes/pool.rs:1-7); typed failures for an id outside the table and for a step that selects
more distinct experts than the pool has rows.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, Iterable, List, Tuple


class ResidencyError(ValueError):
    pass


class ExpertIdOutOfRange(ResidencyError):
    def __init__(self, expert: int, experts: int):
        super().__init__(f"expert id {expert} is not one of the site's {experts} experts")
        self.expert, self.experts = expert, experts


class PoolTooSmall(ResidencyError):
    def __init__(self, needed: int, slots: int):
        super().__init__(f"a step needs {needed} experts but the pool has {slots} rows")
        self.needed, self.slots = needed, slots


@dataclass
class ResidencyCounters:
    syncs: int = 0          # sync points served (all-hit ones included)
    id_reads: int = 0       # expert ids read back across those syncs
    refills: int = 0        # experts written into a pool row
    evictions: int = 0      # refills that displaced another expert
    refill_bytes: int = 0   # device bytes those refills wrote, over every table of the site


@dataclass
class _Site:
    experts: int
    slots: int
    row_expert: List[int] = field(default_factory=list)     # -1 = free
    expert_row: List[int] = field(default_factory=list)     # -1 = not resident
    used: List[int] = field(default_factory=list)           # the sync at which each row was last needed

    def __post_init__(self):
        self.row_expert = [-1] * self.slots
        self.expert_row = [-1] * self.experts
        self.used = [0] * self.slots

    def serve(self, needed: List[int], now: int) -> Tuple[List[Tuple[int, int]], int]:
        """Make ``needed`` (distinct experts) resident at sync ``now``: ``([(row, expert)] to refill, evictions)``."""
        for e in needed:                                    # pin what is resident already: no victim is one of them
            r = self.expert_row[e]
            if r >= 0:
                self.used[r] = now
        fills, evicted = [], 0
        for e in needed:
            if self.expert_row[e] >= 0:
                continue
            row = min((r for r in range(self.slots) if self.used[r] != now),
                      key=lambda r: (self.row_expert[r] >= 0, self.used[r]))
            old = self.row_expert[row]
            if old >= 0:
                self.expert_row[old] = -1
                evicted += 1
            self.row_expert[row], self.expert_row[e], self.used[row] = e, row, now
            fills.append((row, e))
        return fills, evicted


class ExpertResidency:
    """LRU residency per pooled site."""

    def __init__(self):
        self.sites: Dict[Hashable, _Site] = {}
        self.clock = 0
        self.counters = ResidencyCounters()

    def reset(self) -> None:
        """Forget every assignment, the LRU order and the counters, together: called when the device pools were
        cleared or lost (a manager that kept its map would serve stale experts)."""
        self.sites.clear()
        self.clock = 0
        self.counters = ResidencyCounters()

    def sync(self, site: Hashable, ids: Iterable[int], experts: int, slots: int, bytes_per_expert: int = 0):
        """Serve one routed sync point.  Returns ``(fills, map, changed)``: the ``(row, expert)`` refills, the site's
        whole ``[E]`` map from expert id to pool row, and whether the map changed."""
        needed: List[int] = []
        n_ids = 0
        for i in ids:
            i = int(i)
            n_ids += 1
            if i < 0 or i >= experts:
                raise ExpertIdOutOfRange(i, experts)
            if i not in needed:
                needed.append(i)
        if len(needed) > slots:
            raise PoolTooSmall(len(needed), slots)
        self.clock += 1
        st = self.sites.get(site)
        if st is None:
            st = self.sites[site] = _Site(experts, slots)
        if (st.experts, st.slots) != (experts, slots):
            raise ResidencyError(f"site {site!r} was created with {st.experts} experts and {st.slots} rows")
        fills, evicted = st.serve(needed, self.clock)
        c = self.counters
        c.syncs += 1
        c.id_reads += n_ids
        c.refills += len(fills)
        c.evictions += evicted
        c.refill_bytes += len(fills) * bytes_per_expert
        return fills, list(st.expert_row), bool(fills)
