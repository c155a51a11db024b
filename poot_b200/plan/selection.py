"""``form_selection``: the top-k selection of a sparse-attention indexer, formed from the primitive composition a tracer
states.

A tracer writes the selection as ordinary equations - ``keep = not(rank >= k)`` with ``rank = stable_descending_rank(
score)`` - whose middle is quadratic in the number of candidates (every candidate is compared with every other).  No
device runs that; it runs the linear radix select (``csrc/kernels/sparse_index.cu::index_select``).  This pass finds
the composition and folds it, in place, into ONE ``block_top_k`` composite (blocks of one position) whose body is the
composition itself, so the oracle still evaluates it by its decomposition and the planner gives it the select kernel.

Recognition is by the decomposition, never by a hand-written copy of its shape: a candidate root fixes the parameters
(``k``, the score's type), the definition is built over a placeholder of that type with the same ``ir.oplib`` function
the tracer calls, normalised the way ``compile`` normalises the traced graph, and unified with the graph from the
candidate root.  Every equation of the definition must match one of the graph (commutative operands in either order),
so a near-miss - a different tie rule, a changed comparison - is left alone.  (crates/poot-graph-plan/src/passes/
selection.rs:1-25.)
"""
from __future__ import annotations

from typing import Dict, Optional, Set, Tuple

from ..ir import oplib as O
from ..ir.builder import Builder
from ..ir.graph import Graph
from ..tensor import DType
from . import passes
from .edit import Decline, fold_region

COMMUTATIVE = {"add", "mul", "max", "and", "or", "xor"}


def _literal(g: Graph, v: int, by_value) -> Optional[float]:
    """The scalar a value broadcasts, if it is a (broadcast of a) literal."""
    prod = g.producers()
    hops = 0
    while v in prod and g.eqns[prod[v]].op in ("broadcast", "reshape") and hops < 4:
        v, hops = g.eqns[prod[v]].inputs[0], hops + 1
    i = by_value.get(v)
    if i is not None and i.computed and i.computed[0] == "literal":
        return i.computed[1][0]
    return None


def _definition(shape, dtype: DType, k: int) -> Tuple[Graph, int, int]:
    """The selection over a placeholder score: (normalised graph, placeholder value, root value).  ``shape`` is the
    root's: two axes (rows, candidates), or three when the tracer ranks a flattened (rows * tokens, candidates) view
    and shapes the rank back."""
    b = Builder()
    s = b.slot("s", tuple(shape), dtype, "activation")
    if len(shape) == 3:             # the placeholder is the unflattened score: normalisation merges the reshapes around it
        rank = b.reshape(O.stable_descending_rank(b, b.reshape(s, (shape[0] * shape[1], shape[2]))), tuple(shape))
    else:
        rank = O.stable_descending_rank(b, s)
    keep = O.lnot(b, b.binary("ge", rank, b.broadcast(b.scalar(k, DType.I32), rank.shape)))
    b.output(keep, "keep", "result")
    d = b.finish()
    passes.canonicalize(d)
    passes.cse(d)
    return d, d.inputs[0].value, d.outputs[0].value


def _unify(d: Graph, g: Graph, dv: int, gv: int, bind: Dict[int, int], region: Set[int], dprod, gprod, dby, gby,
           placeholder: int) -> bool:
    if dv in bind:
        return bind[dv] == gv
    if d.types[dv] != g.types[gv]:
        return False
    if dv == placeholder:
        bind[dv] = gv
        return True
    di = dby.get(dv)
    if di is not None:                          # a literal / computed input of the definition
        gi = gby.get(gv)
        if gi is None or gi.computed != di.computed:
            return False
        bind[dv] = gv
        return True
    dk, gk = dprod.get(dv), gprod.get(gv)
    if dk is None or gk is None:
        return False
    de, ge = d.eqns[dk], g.eqns[gk]
    if de.op != ge.op or len(de.inputs) != len(ge.inputs) or de.attrs != ge.attrs or len(ge.outputs) != 1:
        return False
    orders = [list(ge.inputs)]
    if de.op in COMMUTATIVE and len(ge.inputs) == 2:
        orders.append(list(reversed(ge.inputs)))
    for order in orders:
        trial, tregion = dict(bind), set(region)
        trial[dv] = gv
        tregion.add(gk)
        if all(_unify(d, g, a, b_, trial, tregion, dprod, gprod, dby, gby, placeholder) for a, b_ in zip(de.inputs, order)):
            bind.clear(); bind.update(trial)
            region.clear(); region.update(tregion)
            return True
    return False


def form_selection(g: Graph, declines: Optional[list] = None) -> int:
    """Fold every ``not(stable_descending_rank(score) >= k)`` into a ``block_top_k`` composite; returns how many."""
    n = 0
    tried: Set[int] = set()
    while True:
        gprod = g.producers()
        gby = {i.value: i for i in g.inputs}
        found = None
        for ei, e in enumerate(g.eqns):
            if e.op != "xor" or e.outputs[0] in tried or len(g.types[e.outputs[0]].shape) not in (2, 3):
                continue
            # root shape: xor(ge(rank, k...), 1...) in either operand order
            for a in e.inputs:
                j = gprod.get(a)
                if j is None or g.eqns[j].op != "ge":
                    continue
                k = _literal(g, g.eqns[j].inputs[1], gby)
                if k is None or int(k) != k or k < 1:
                    continue
                rank = g.eqns[j].inputs[0]
                r = gprod.get(rank)
                if r is not None and g.eqns[r].op == "reshape":
                    r = gprod.get(g.eqns[r].inputs[0])
                if r is None or g.eqns[r].op != "reduce":
                    continue
                # the score is whatever the definition's placeholder binds to: try to unify from the root
                shape = g.types[e.outputs[0]].shape
                for dt in (DType.F32,):
                    d, ph, root = _definition(shape, dt, int(k))
                    bind: Dict[int, int] = {}
                    region: Set[int] = set()
                    dby = {i.value: i for i in d.inputs}
                    if _unify(d, g, root, e.outputs[0], bind, region, d.producers(), gprod, dby, gby, ph):
                        found = (region, {"k": int(k), "ratio": 1, "tie": "lowest_index"}, bind[ph], ei)
                        break
                if found:
                    break
            if found:
                break
            if e.op == "xor":
                tried.add(e.outputs[0])
        if found is None:
            return n
        region, attrs, score, ei = found
        # What does not depend on the score - the index grids and the "lower index" predicate built from them - is shared
        # by every selection of the graph after CSE: it stays outside and enters the composite as operands, which no
        # kernel materialises.
        dep = {score}
        for k in sorted(region):
            if any(v in dep for v in g.eqns[k].inputs):
                dep.update(g.eqns[k].outputs)
        region = {k for k in region if any(v in dep for v in g.eqns[k].inputs)}
        try:
            fold_region(g, region, "block_top_k", attrs)
            n += 1
        except Decline as dcl:
            (declines if declines is not None else []).append(("block_top_k", ei, str(dcl)))
            tried.add(g.eqns[ei].outputs[0])
