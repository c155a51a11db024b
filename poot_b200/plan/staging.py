"""Stage split: cut a step graph into consecutive stage graphs joined by boundary descriptors
(crates/poot-graph-plan/src/passes/stage_split.rs:1-8,220-255; src/staged.rs:137-260).

Values that cross a cut become ``export`` outputs of the producing stage and device inputs of the consuming one;
each stage keeps the constants, slots and carried state its own equations touch.  Running the stages in order and
handing the boundary values across reproduces the whole graph exactly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

from ..ir.graph import Eqn, Graph, Input, Output


@dataclass
class Boundary:
    name: str
    value: int
    nbytes: int
    producer: int      # stage index
    consumers: List[int]


def split_stages(g: Graph, cuts: Sequence[int]) -> (List[Graph], List[Boundary]):
    """``cuts``: equation indices where a new stage starts (ascending)."""
    edges = [0] + list(cuts) + [len(g.eqns)]
    if sorted(set(edges)) != edges:
        raise ValueError("cuts must be ascending equation indices inside the graph")
    stage_of: Dict[int, int] = {}
    for s in range(len(edges) - 1):
        for k in range(edges[s], edges[s + 1]):
            for v in g.eqns[k].outputs:
                stage_of[v] = s
    in_by_value = {i.value: i for i in g.inputs}
    bounds: Dict[int, Boundary] = {}
    stages: List[Graph] = []
    for s in range(len(edges) - 1):
        sg = Graph()
        sg.types, sg.names, sg._next = dict(g.types), dict(g.names), g._next
        eqns = g.eqns[edges[s]:edges[s + 1]]
        needed = []
        for e in eqns:
            for v in e.inputs:
                if v not in needed and stage_of.get(v, -1) != s:
                    needed.append(v)
        out_vals = [o for o in g.outputs if stage_of.get(o.value, -1) == s or
                    (o.value in in_by_value and s == len(edges) - 2)]
        for v in needed:
            if v in in_by_value:
                sg.inputs.append(Input(**vars(in_by_value[v])))
            else:
                b = bounds[v]
                b.consumers.append(s)
                sg.inputs.append(Input(v, b.name, storage="device"))
        sg.eqns = [Eqn(e.op, list(e.inputs), list(e.outputs), dict(e.attrs), e.body) for e in eqns]
        sg.outputs = [Output(**vars(o)) for o in out_vals]
        # values defined here and used by a later stage
        later_use = set()
        for k in range(edges[s + 1], len(g.eqns)):
            later_use.update(g.eqns[k].inputs)
        for e in eqns:
            for v in e.outputs:
                if v in later_use:
                    b = Boundary(f"boundary.{v}", v, g.types[v].nbytes, s, [])
                    bounds[v] = b
                    if not any(o.value == v for o in sg.outputs):
                        sg.outputs.append(Output(v, b.name, "export"))
                    else:
                        sg.outputs.append(Output(v, b.name, "export"))
        sg.validate()
        stages.append(sg)
    return stages, list(bounds.values())
