"""LoRA as a graph transform: every targeted projection ``y = x W^T`` becomes
``y + scale[idx] * IndexedMatMul(IndexedMatMul(x, A, idx), B, idx)`` with a per-row adapter index
(crates/poot-graph-plan/src/passes/lora.rs:1-7).  Index 0 is "no adapter" (all-zero factors), so one captured step
serves rows that use different adapters.  The device engine does not run this form (it merges one adapter at load,
see ``load/lora.py``); the transform exists so the oracle defines what per-request adapters mean and so the two
forms can be checked against each other.
"""
from __future__ import annotations

from typing import Dict, List

from ..ir.graph import Eqn, Graph, Input, TensorType
from ..tensor import DType


def lora_targets(g: Graph) -> Dict[str, int]:
    """canonical weight name -> index of the matmul equation that applies it (``matmul(x, transpose(cast?(W)))``)."""
    prod = g.producers()
    by_value = {i.value: i for i in g.inputs}
    out = {}
    for k, e in enumerate(g.eqns):
        if e.op != "matmul" or e.inputs[1] not in prod:
            continue
        t = g.eqns[prod[e.inputs[1]]]
        if t.op != "transpose":
            continue
        v = t.inputs[0]
        while v in prod and g.eqns[prod[v]].op == "cast":
            v = g.eqns[prod[v]].inputs[0]
        inp = by_value.get(v)
        if inp is not None and inp.storage == "const" and g.types[v].rank == 2:
            out[inp.name] = k
    return out


def apply_lora(g: Graph, targets: List[str], rank: int, adapters: int) -> Graph:
    """Returns a new graph with inputs ``lora.idx`` [rows] (slot), ``lora.scale`` [adapters + 1] and, per target,
    ``<name>.lora_a`` [adapters + 1, in, rank] / ``<name>.lora_b`` [adapters + 1, rank, out]."""
    where = lora_targets(g)
    missing = [t for t in targets if t not in where]
    if missing:
        raise ValueError(f"no projection applies {missing}")
    by_eqn = {where[t]: t for t in targets}
    new = Graph()
    new.types, new.names, new._next = dict(g.types), dict(g.names), g._next
    new.inputs = [Input(**vars(i)) for i in g.inputs]
    new.outputs = list(g.outputs)
    n_slots = adapters + 1
    idx = scale = None
    rep: Dict[int, int] = {}
    for k, e in enumerate(g.eqns):
        ins = [rep.get(v, v) for v in e.inputs]
        new.eqns.append(Eqn(e.op, ins, list(e.outputs), dict(e.attrs), e.body))
        if k not in by_eqn:
            continue
        name = by_eqn[k]
        x, y = ins[0], e.outputs[0]
        M, Kd = g.types[x].shape
        N = g.types[y].shape[1]
        if idx is None:
            idx = new.add_input("lora.idx", TensorType((M,), DType.I32), storage="slot", slot="owned", range=(0, adapters))
            scale = new.add_input("lora.scale", TensorType((n_slots,), DType.F32), storage="const")
        a = new.add_input(f"{name}.lora_a", TensorType((n_slots, Kd, rank), DType.F32), storage="const")
        b = new.add_input(f"{name}.lora_b", TensorType((n_slots, rank, N), DType.F32), storage="const")
        (xa,) = new.add_eqn("indexed_matmul", [x, a, idx], {"precision": e.attrs.get("precision", "narrow")})
        (xab,) = new.add_eqn("indexed_matmul", [xa, b, idx], {"precision": e.attrs.get("precision", "narrow")})
        (srow,) = new.add_eqn("gather", [scale, idx], {"axis": 0})
        (scol,) = new.add_eqn("reshape", [srow], {"shape": (M, 1)})
        (sb,) = new.add_eqn("broadcast", [scol], {"shape": (M, N)})
        (delta,) = new.add_eqn("mul", [xab, sb])
        (y2,) = new.add_eqn("add", [y, delta])
        rep[y] = y2
    for o in new.outputs:
        o.value = rep.get(o.value, o.value)
    new.validate()
    return new
