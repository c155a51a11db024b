"""How a step's carried state is committed (crates/poot-graph-plan/src/state_commit.rs:1-7).

A graph's state transition is a simultaneous assignment: every ``state_next`` output is computed from the step's
``state`` inputs as they were when the step began.  An executor may let the equation that materialises a next state
overwrite the state input's own buffer (donation) only when that cannot change anything the graph still reads: the input
(through casts to its own type, which are the same buffer) must have no reader other than that equation, the equation
must be an update that leaves the untouched elements as they were (``scatter_update`` / ``dynamic_update_slice`` with the
state as its base), and no other state may be computed from the old contents.  Every other state is committed by copying
its next value into place after the equations have run.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

from ..ir.graph import Graph

UPDATES = ("scatter_update", "dynamic_update_slice")


@dataclass
class StateCommitPlan:
    inplace: Dict[int, str] = field(default_factory=dict)      # equation index -> state input it overwrites in place
    copies: List[tuple] = field(default_factory=list)           # (state input name, output name) committed after the step
    reasons: Dict[str, str] = field(default_factory=dict)       # state input name -> why it is copied


def plan_state_commit(g: Graph) -> StateCommitPlan:
    plan = StateCommitPlan()
    users = g.users()
    prod = g.producers()
    outs_by_state = {o.state_of: o for o in g.outputs if o.role == "state_next"}
    for i in g.inputs:
        if i.storage != "state" or i.name not in outs_by_state:
            continue
        out = outs_by_state[i.name]
        # the state's buffer under casts that keep its type
        alias, frontier = {i.value}, [i.value]
        while frontier:
            v = frontier.pop()
            for u in users.get(v, []):
                e = g.eqns[u]
                if e.op == "cast" and g.types[e.outputs[0]] == g.types[v] and e.outputs[0] not in alias:
                    alias.add(e.outputs[0])
                    frontier.append(e.outputs[0])
        readers = {u for v in alias for u in users.get(v, []) if not (g.eqns[u].op == "cast" and g.eqns[u].outputs[0] in alias)}
        # the next value, back through casts that keep the type
        nv = out.value
        while nv in prod and g.eqns[prod[nv]].op == "cast" and g.types[g.eqns[prod[nv]].inputs[0]] == g.types[nv]:
            nv = g.eqns[prod[nv]].inputs[0]
        k = prod.get(nv)
        why = None
        if k is None or g.eqns[k].op not in UPDATES:
            why = "the next value is not an in-place update of the state"
        elif g.eqns[k].inputs[0] not in alias:
            why = "the update's base is not this state"
        elif readers != {k}:
            why = "the old contents are read by another equation"
        if why is None:
            plan.inplace[k] = i.name
        else:
            plan.copies.append((i.name, out.name))
            plan.reasons[i.name] = why
    return plan
