"""Graph surgery shared by the passes: fold a set of equations into one composite that carries them as its body.

The composite keeps the value ids of the region's live-out values, so every user outside the region stays valid,
and its body is the region verbatim - the oracle evaluates the rewritten graph through exactly the primitives the
tracer emitted (crates/poot-graph-ir/src/graph.rs:1361-1960 `GraphEdit`).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Set

from ..ir.graph import Eqn, Graph


class Decline(Exception):
    """A matcher found its anchor but the surrounding graph does not allow the rewrite; recorded, not raised further."""


def fold_region(g: Graph, idxs: Iterable[int], op: str, attrs: Optional[dict] = None,
                input_order: Optional[List[int]] = None) -> Eqn:
    """Replace equations ``idxs`` of ``g`` (in place) by one composite ``op``; returns the new equation."""
    region = sorted(set(idxs))
    if not region:
        raise Decline("empty region")
    # a shaping equation (broadcast / reshape of an outside value) that other equations share stays outside
    users0 = g.users()
    changed = True
    while changed:
        changed = False
        rs = set(region)
        made_by = {v: k for k in region for v in g.eqns[k].outputs}
        for k in list(region):
            e = g.eqns[k]
            if e.op not in ("broadcast", "reshape") or not any(u not in rs for u in users0.get(e.outputs[0], [])):
                continue
            # its operands come from outside, or from shaping equations of the region (which then leave with it)
            if all(v not in made_by or g.eqns[made_by[v]].op in ("broadcast", "reshape") for v in e.inputs):
                region.remove(k)
                changed = True
                break
    inside: Set[int] = set()
    for k in region:
        inside.update(g.eqns[k].outputs)
    ext: List[int] = []
    for k in region:
        for v in g.eqns[k].inputs:
            if v not in inside and v not in ext:
                ext.append(v)
    if input_order is not None:
        if set(input_order) != set(ext):
            raise Decline("region inputs differ from the matcher's operands")
        ext = list(input_order)
    rset = set(region)
    users = g.users()
    graph_outs = {o.value for o in g.outputs}
    last = region[-1]
    live_out: List[int] = []
    for k in region:
        for v in g.eqns[k].outputs:
            outside = [u for u in users.get(v, []) if u not in rset]
            if outside or v in graph_outs:
                if any(u < last for u in outside):
                    raise Decline("a region value is used before the region ends")
                live_out.append(v)
    if not live_out:
        raise Decline("region has no live output")
    body = Graph()
    m: Dict[int, int] = {}
    for i, v in enumerate(ext):
        m[v] = body.add_input(f"in{i}", g.types[v])
    for k in region:
        e = g.eqns[k]
        outs = body.add_eqn(e.op, [m[v] for v in e.inputs], e.attrs, e.body)
        for a, b_ in zip(e.outputs, outs):
            m[a] = b_
    for i, v in enumerate(live_out):
        body.add_output(m[v], f"out{i}")
    new = Eqn(op, ext, live_out, dict(attrs or {}), body)
    eqns: List[Eqn] = []
    for k, e in enumerate(g.eqns):
        if k == last:
            eqns.append(new)
        elif k not in rset:
            eqns.append(e)
    g.eqns = eqns
    return new


def literal_value(g: Graph, v: int):
    """Value of a literal scalar input (or of a broadcast of one), else None."""
    prod = g.producers()
    while v in prod and g.eqns[prod[v]].op in ("broadcast", "reshape"):
        v = g.eqns[prod[v]].inputs[0]
    for i in g.inputs:
        if i.value == v and i.computed and i.computed[0] == "literal":
            return i.computed[1][0]
    return None


def sole_user(users: Dict[int, List[int]], v: int, graph_outs: Set[int]) -> Optional[int]:
    u = users.get(v, [])
    return u[0] if len(u) == 1 and v not in graph_outs else None
