"""Static analyses over a graph (crates/poot-graph-ir/src/analysis/stats.rs:13,72, src/range.rs:186,
src/index_guard.rs:102, src/slot_map.rs).

* ``dispatch_count``: equations that cost a launch when nothing is fused (movement that is a pure view is free).
* ``peak_transient_bytes``: the largest number of bytes of computed values alive at once, walking the equations in
  order (inputs and outputs excluded: they are owned by the caller).
* ``value_ranges``: interval analysis of the I32 values, seeded by the declared ranges of the slots; the index
  guards are read off it.
* ``index_guards``: for every gather / scatter, whether its indices are PROVEN inside the indexed extent; an
  unproven one needs a device witness (or is refused), never a silent clamp.
* ``check_write_slots``: duplicate write slots are refused before launch (a scatter with duplicate targets is a race).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..tensor import DType
from .graph import Graph

FREE = {"reshape"}
Interval = Tuple[int, int]


def dispatch_count(g: Graph) -> int:
    return sum(1 for e in g.eqns if e.op not in FREE)


def peak_transient_bytes(g: Graph) -> int:
    last_use: Dict[int, int] = {}
    for k, e in enumerate(g.eqns):
        for v in e.inputs:
            last_use[v] = k
    outs = {o.value for o in g.outputs}
    alive = 0
    peak = 0
    dying: Dict[int, List[int]] = {}
    for k, e in enumerate(g.eqns):
        for v in e.outputs:
            if v in outs:
                continue
            alive += g.types[v].nbytes
            dying.setdefault(last_use.get(v, k), []).append(v)
        peak = max(peak, alive)
        for v in dying.pop(k, []):
            alive -= g.types[v].nbytes
    return peak


def _mul(a: Interval, b: Interval) -> Interval:
    c = [a[0] * b[0], a[0] * b[1], a[1] * b[0], a[1] * b[1]]
    return min(c), max(c)


def value_ranges(g: Graph) -> Dict[int, Interval]:
    """value id -> inclusive [lo, hi] for I32 values whose range is known."""
    r: Dict[int, Interval] = {}
    for i in g.inputs:
        ty = g.types[i.value]
        if ty.dtype != DType.I32:
            continue
        if i.range is not None:
            r[i.value] = (int(i.range[0]), int(i.range[1]))
        elif i.computed and i.computed[0] == "literal":
            v = int(i.computed[1][0])
            r[i.value] = (v, v)
    for e in g.eqns:
        ins = [r.get(v) for v in e.inputs]
        out = e.outputs[0] if e.outputs else None
        if out is None or g.types[out].dtype != DType.I32:
            continue
        op = e.op
        if op in ("reshape", "broadcast", "transpose", "slice", "cast") and ins[0] is not None:
            r[out] = ins[0]
        elif op == "concat" and all(x is not None for x in ins):
            r[out] = (min(x[0] for x in ins), max(x[1] for x in ins))
        elif op == "iota":
            r[out] = (0, e.attrs["shape"][e.attrs["axis"]] - 1)
        elif op == "reduce" and e.attrs.get("kind", "sum") == "max" and ins[0] is not None:
            r[out] = ins[0]
        elif op in ("add", "sub", "mul", "max") and ins[0] is not None and ins[1] is not None:
            a, b = ins
            if op == "add":
                r[out] = (a[0] + b[0], a[1] + b[1])
            elif op == "sub":
                r[out] = (a[0] - b[1], a[1] - b[0])
            elif op == "mul":
                r[out] = _mul(a, b)
            else:
                r[out] = (max(a[0], b[0]), max(a[1], b[1]))
        elif op in ("ge", "geu", "and", "or", "xor", "not") and all(x is not None and 0 <= x[0] and x[1] <= 1 for x in ins):
            r[out] = (0, 1)
        elif op == "ge":
            r[out] = (0, 1)
        elif op == "remu" and ins[1] is not None and ins[1][0] > 0:
            r[out] = (0, ins[1][1] - 1)
        elif op == "shr" and ins[0] is not None and ins[1] is not None and ins[0][0] >= 0 and ins[1][0] >= 0:
            r[out] = (ins[0][0] >> ins[1][1], ins[0][1] >> ins[1][0])
        elif op == "select" and ins[1] is not None and ins[2] is not None:
            r[out] = (min(ins[1][0], ins[2][0]), max(ins[1][1], ins[2][1]))
        elif op == "gather" and ins[0] is not None:
            r[out] = ins[0]                      # elements of an I32 table keep the table's range
        elif op == "arg_top_k":
            n = g.types[e.inputs[0]].shape[-1]
            r[out] = (0, n - 1)
        elif op == "ngram_hash":                 # every head's id lies in its own slice of the table
            at = e.attrs
            r[out] = (min(at["offsets"]), max(o + p_ - 1 for o, p_ in zip(at["offsets"], at["primes"])))
    return r


@dataclass
class IndexGuard:
    eqn: int
    op: str
    extent: int
    range: Optional[Interval]
    proven: bool
    allows_skip: bool = False        # scatter_update treats -1 as "write nothing"


def index_guards(g: Graph) -> List[IndexGuard]:
    r = value_ranges(g)
    out: List[IndexGuard] = []
    for k, e in enumerate(g.eqns):
        if e.op == "gather":
            extent = g.types[e.inputs[0]].shape[e.attrs.get("axis", 0)]
            iv = r.get(e.inputs[1])
            out.append(IndexGuard(k, "gather", extent, iv, iv is not None and iv[0] >= 0 and iv[1] < extent))
        elif e.op == "scatter_update":
            extent = g.types[e.inputs[0]].shape[0]
            iv = r.get(e.inputs[1])
            out.append(IndexGuard(k, "scatter_update", extent, iv, iv is not None and iv[0] >= -1 and iv[1] < extent, True))
        elif e.op == "indexed_matmul":
            extent = g.types[e.inputs[1]].shape[0]
            iv = r.get(e.inputs[2])
            out.append(IndexGuard(k, "indexed_matmul", extent, iv, iv is not None and iv[0] >= 0 and iv[1] < extent))
    return out


class DuplicateWriteSlot(ValueError):
    pass


def check_write_slots(write_map: np.ndarray) -> None:
    """Host-side check before launch: every slot other than -1 (skip) may be written at most once per step."""
    w = np.asarray(write_map).reshape(-1)
    live = w[w >= 0]
    if live.size and np.unique(live).size != live.size:
        vals, counts = np.unique(live, return_counts=True)
        raise DuplicateWriteSlot(f"slot {int(vals[counts > 1][0])} is written {int(counts.max())} times in one step")


# ---- numerics classes ---------------------------------------------------------------------------------------------------
NUMERICS_ORDER = ("exact", "unfused", "reassociating", "narrowing")
# comparison tolerance of a device result against the oracle, relative to max(|oracle element|, 1), by the strongest
# property the compiled program exhibits (crates/poot-graph-ir/src/analysis/numerics.rs:83-96)
TIER2_TOLERANCE = {"exact": 0.0, "unfused": 1e-4, "reassociating": 1e-3, "narrowing": 5e-3}
_REASSOCIATING_OPS = {"attention", "rope", "fused", "fused_row", "contraction_epilogue", "dense_contraction", "grouped_dense_contraction",
                      "expert_group", "block_top_k", "selected_attention"}
_NARROWING_OPS = {"packed_contraction", "packed_row_gather", "packed_dequant"}
_FLOAT_ARITHMETIC = {"add", "sub", "mul", "div", "max", "neg", "exp", "log", "sqrt", "recip", "tanh", "erf", "reduce", "matmul",
                     "indexed_matmul", "scan", "all_reduce"}


def implied_numerics(g: Graph) -> str:
    """The strongest numerics property the graph's equations imply, in ``NUMERICS_ORDER``: ``exact`` (integer and
    movement equations only), ``unfused`` (ordinary float arithmetic a device runs as written), ``reassociating`` (a
    composite that reorders float arithmetic: fusion, tiling, flash attention, rope) or ``narrowing`` (a quantised
    decode, a contraction whose operands are rounded to a 16-bit type, a float value stored narrower than f32).  It
    describes how closely a device result can be expected to follow the oracle (``TIER2_TOLERANCE``), not whether a
    rewrite is legal."""
    rank = 0
    for e in g.eqns:
        out = g.types[e.outputs[0]] if e.outputs else None
        r = 0
        if e.op in _NARROWING_OPS or (e.op in ("matmul", "indexed_matmul", "dense_contraction", "packed_contraction", "attention")
                                      and e.attrs.get("precision", "narrow") != "exact"):
            r = 3
        elif e.op == "cast" and e.attrs["dtype"].is_float and e.attrs["dtype"].size < 4:
            r = 3
        elif e.op in _REASSOCIATING_OPS:
            r = 2
        elif e.op in _FLOAT_ARITHMETIC and out is not None and out.dtype.is_float:
            r = 1
        if e.body is not None:
            r = max(r, NUMERICS_ORDER.index(implied_numerics(e.body)))
        rank = max(rank, r)
    return NUMERICS_ORDER[rank]
