"""Preparation passes that run between the matchers and the fusion passes: they change how a value is produced, never
what it is.

* ``fold_iota``: an ``iota`` equation has a static shape and no operands, so its value is known when the graph is
  compiled.  It becomes a computed constant (``("iota", (axis,))``) that the executor materialises once, like a rope
  table, instead of a launch per step; equal iotas share one constant (crates/poot-graph-plan/src/passes/iota.rs:1-26).
  It runs after the attention, selection and recurrent-block matchers, which recognise masks by their iota equations.
* ``lower_nonlast_reduces``: a ``reduce`` over an axis that is not the last one becomes transpose -> reduce over the
  last axis (-> reshape when the axis is kept), so that the row kernels, which reduce along contiguous rows, are the
  only reduction the planner has to place (crates/poot-graph-plan/src/dtype_widen.rs:600-622).  The sum runs over the
  same elements in the same order, so the result is bit-identical.

Mixed operand types need no widening pass here: the graph's typing rules refuse a binary equation, a select or a concat
whose operands differ in type when the tracer emits it, so a graph that reaches the planner has every widening written
as a ``cast`` already, and the fusion passes absorb those casts into the regions that read them.
"""
from __future__ import annotations

from typing import Dict

from ..ir.graph import Eqn, Graph, Input, TensorType
from ..tensor import DType


def fold_iota(g: Graph) -> int:
    """Every top-level ``iota`` becomes a computed constant; returns how many equations were folded."""
    made: Dict[tuple, int] = {}
    rep: Dict[int, int] = {}
    keep = []
    taken = {i.name for i in g.inputs}
    for e in g.eqns:
        if e.op != "iota":
            keep.append(e)
            continue
        shape, axis, dtype = tuple(e.attrs["shape"]), int(e.attrs["axis"]), e.attrs.get("dtype", DType.I32)
        key = (shape, axis, dtype)
        if key in made:
            rep[e.outputs[0]] = made[key]
            continue
        name = f"iota.{'x'.join(map(str, shape))}.{axis}.{dtype}"
        while name in taken:
            name += "_"
        taken.add(name)
        v = e.outputs[0]                       # the value keeps its id: readers need no rewiring
        g.names[v] = name
        g.inputs.append(Input(v, name, storage="computed", computed=("iota", (axis,)),
                              range=(0, shape[axis] - 1) if dtype == DType.I32 else None))
        made[key] = v
    folded = len(g.eqns) - len(keep)
    g.eqns = keep
    if rep:
        for e in g.eqns:
            e.inputs = [rep.get(v, v) for v in e.inputs]
        for o in g.outputs:
            o.value = rep.get(o.value, o.value)
    return folded


def lower_nonlast_reduces(g: Graph) -> int:
    """Every top-level ``reduce`` over a non-last axis is rewritten to reduce over the last axis of a transposed view.
    The reduce's own output value is kept, so named outputs and state bindings survive."""
    out = []
    n = 0
    for e in g.eqns:
        x = e.inputs[0] if e.inputs else None
        if e.op != "reduce" or g.types[x].rank < 2:
            out.append(e)
            continue
        ty = g.types[x]
        ax = e.attrs["axis"] % ty.rank
        if ax == ty.rank - 1:
            out.append(e)
            continue
        perm = tuple(i for i in range(ty.rank) if i != ax) + (ax,)
        moved = g.new_value(TensorType(tuple(ty.shape[p] for p in perm), ty.dtype))
        out.append(Eqn("transpose", [x], [moved], {"perm": perm}))
        keep = bool(e.attrs.get("keepdim", False))
        if keep:
            flat = g.new_value(TensorType(tuple(ty.shape[p] for p in perm[:-1]), ty.dtype))
            out.append(Eqn("reduce", [moved], [flat], {**e.attrs, "axis": ty.rank - 1, "keepdim": False}))
            out.append(Eqn("reshape", [flat], list(e.outputs), {"shape": tuple(g.types[e.outputs[0]].shape)}))
        else:
            out.append(Eqn("reduce", [moved], list(e.outputs), {**e.attrs, "axis": ty.rank - 1, "keepdim": False}))
        n += 1
    g.eqns = out
    return n
