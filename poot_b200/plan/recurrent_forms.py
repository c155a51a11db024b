"""``form_recurrent_blocks``: the two compositions around a recurrent mixer's scan that have kernels of their own.

* ``causal_conv_silu``: ``silu(causal_conv1d(state ++ x, taps [+ bias]))`` over one sequence row - the depthwise causal
  convolution a tracer writes as ``K`` shifted slices times broadcast taps - with the window it hands on
  (``csrc/kernels/gdn.cu::causal_conv_silu_kernel`` does the conv, the activation and the window update in one launch);
* ``gated_rmsnorm``: ``rmsnorm(y, w) * act(z)`` or ``rmsnorm(y * silu(z), w)`` per head
  (``csrc/kernels/gdn.cu::gated_rmsnorm_kernel``).

Recognition is by the decomposition, as in ``selection.py``: the definition is built over placeholders with the same
``ir.oplib`` function the tracers call, normalised like the traced graph and unified with the graph from a candidate
root.  A literal of the definition marked as a parameter (the norm's epsilon) binds to whatever literal the graph has at
that place.  Every equation of the definition must match, so a conv with another tap order or a norm gated some other
way stays as primitives.  The composite's body is the matched region, so the oracle evaluates it unchanged
(crates/poot-graph-plan/src/passes/: the reference forms its scan neighbours during staging).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Set, Tuple

from ..ir import oplib as O
from ..ir.builder import Builder
from ..ir.graph import Graph
from ..tensor import DType
from . import passes
from .edit import Decline, fold_region

COMMUTATIVE = {"add", "mul", "max", "and", "or", "xor"}
EPS_SENTINEL = 0.12345678          # stands for "some epsilon" inside a definition


class Definition:
    """A normalised definition graph with named placeholders and the value that is its root."""

    def __init__(self, build: Callable[[Builder, Dict[str, object]], object], slots: Dict[str, tuple]):
        b = Builder()
        ph = {n: b.slot(n, shape, DType.F32, "activation") for n, shape in slots.items()}
        root = build(b, ph)
        b.output(root, "root", "result")
        self.g = b.finish()
        passes.canonicalize(self.g)
        passes.cse(self.g)
        self.placeholders = {i.value: i.name for i in self.g.inputs if i.name in slots}
        self.root = self.g.outputs[0].value
        self.prod = self.g.producers()
        self.by_value = {i.value: i for i in self.g.inputs}


def unify(d: Definition, g: Graph, dv: int, gv: int, bind: Dict[int, int], region: Set[int], params: Dict[str, float], gprod, gby) -> bool:
    if dv in bind:
        return bind[dv] == gv
    if d.g.types[dv] != g.types[gv]:
        return False
    if dv in d.placeholders:
        bind[dv] = gv
        return True
    di = d.by_value.get(dv)
    if di is not None:                                   # a literal / computed input of the definition
        gi = gby.get(gv)
        if gi is None or not gi.computed or not di.computed or gi.computed[0] != di.computed[0]:
            return False
        if di.computed[0] == "literal" and abs(di.computed[1][0] - EPS_SENTINEL) < 1e-9:
            val = gi.computed[1][0]
            if params.setdefault("eps", val) != val:
                return False
        elif gi.computed != di.computed:
            return False
        bind[dv] = gv
        return True
    dk, gk = d.prod.get(dv), gprod.get(gv)
    if dk is None or gk is None:
        return False
    de, ge = d.g.eqns[dk], g.eqns[gk]
    if de.op != ge.op or len(de.inputs) != len(ge.inputs) or de.attrs != ge.attrs or len(ge.outputs) != len(de.outputs):
        return False
    if len(ge.outputs) != 1:
        return False
    orders = [list(ge.inputs)]
    if de.op in COMMUTATIVE and len(ge.inputs) == 2:
        orders.append(list(reversed(ge.inputs)))
    for order in orders:
        tb, tr, tp = dict(bind), set(region), dict(params)
        tb[dv] = gv
        tr.add(gk)
        if all(unify(d, g, a, b_, tb, tr, tp, gprod, gby) for a, b_ in zip(de.inputs, order)):
            bind.clear(); bind.update(tb)
            region.clear(); region.update(tr)
            params.clear(); params.update(tp)
            return True
    return False


def _conv_definition(L: int, C: int, K: int, bias: bool) -> Definition:
    slots = {"x": (L, C), "state": (K - 1, C), "w": (C, K)}
    if bias:
        slots["bias"] = (C,)
    return Definition(lambda b, p: O.silu(b, O.causal_conv1d(b, p["x"], p["state"], p["w"], p.get("bias"))[0]), slots)


def _gated_norm_definition(shape, wshape, gate_first: bool, act: str) -> Definition:
    return Definition(lambda b, p: O.gated_rmsnorm(b, p["y"], p["z"], p["w"], EPS_SENTINEL, gate_first, act),
                      {"y": tuple(shape), "z": tuple(shape), "w": tuple(wshape)})


def _grouped_gate_first_definition(shape) -> Definition:
    """Mamba2's form: the gate is applied on the flat channels, the norm runs within each of the channel groups."""
    L, G, P = shape
    return Definition(lambda b, p: O.rmsnorm(b, b.reshape(p["y"] * O.silu(b, p["z"]), (L, G, P)), b.reshape(p["w"], (G, P)), EPS_SENTINEL),
                      {"y": (L, G * P), "z": (L, G * P), "w": (G * P,)})


def form_recurrent_blocks(g: Graph, declines: Optional[list] = None) -> Dict[str, int]:
    """Fold every conv + SiLU and every gated norm of the graph into its composite; returns how many of each."""
    out = {"causal_conv_silu": 0, "gated_rmsnorm": 0}
    tried: Set[Tuple[str, int]] = set()
    cache: Dict[tuple, Definition] = {}
    while True:
        gprod = g.producers()
        gby = {i.value: i for i in g.inputs}
        found = None
        for ei, e in enumerate(g.eqns):
            shape = tuple(g.types[e.outputs[0]].shape) if e.outputs else ()
            if e.op == "div" and len(shape) == 2 and ("conv", e.outputs[0]) not in tried:
                tried.add(("conv", e.outputs[0]))
                L, C = shape
                for K in (4, 3, 2):
                    for bias in (False, True):
                        key = ("conv", L, C, K, bias)
                        d = cache.get(key) or cache.setdefault(key, _conv_definition(L, C, K, bias))
                        bind, region, params = {}, set(), {}
                        if unify(d, g, d.root, e.outputs[0], bind, region, params, gprod, gby):
                            # the window the conv hands on is a slice of the same ``state ++ x``: it leaves with the conv
                            users = g.users()
                            for k in [k for k in region if g.eqns[k].op == "concat"]:
                                region |= {u for u in users.get(g.eqns[k].outputs[0], []) if g.eqns[u].op == "slice"}
                            found = ("causal_conv_silu", region, {"taps": K, "bias": bias})
                            break
                    if found:
                        break
            elif e.op == "mul" and len(shape) == 3 and ("norm", e.outputs[0]) not in tried:
                tried.add(("norm", e.outputs[0]))
                for wshape in (shape[-1:], shape[-2:]):
                    for gate_first, act in ((False, "silu"), (False, "sigmoid"), (True, "silu")):
                        key = ("norm", shape, wshape, gate_first, act)
                        d = cache.get(key) or cache.setdefault(key, _gated_norm_definition(shape, wshape, gate_first, act))
                        bind, region, params = {}, set(), {}
                        if unify(d, g, d.root, e.outputs[0], bind, region, params, gprod, gby) and "eps" in params:
                            found = ("gated_rmsnorm", region, {"eps": params["eps"], "gate_first": gate_first, "act": act})
                            break
                    if found:
                        break
                if not found:
                    key = ("norm-grouped", shape)
                    d = cache.get(key) or cache.setdefault(key, _grouped_gate_first_definition(shape))
                    bind, region, params = {}, set(), {}
                    if unify(d, g, d.root, e.outputs[0], bind, region, params, gprod, gby) and "eps" in params:
                        found = ("gated_rmsnorm", region, {"eps": params["eps"], "gate_first": True, "act": "silu", "groups": shape[1]})
            if found:
                break
        if found is None:
            return out
        op, region, attrs = found
        try:
            fold_region(g, region, "fused_row", {"kind": op, **attrs})
            out[op] += 1
        except Decline as dcl:
            (declines if declines is not None else []).append((op, min(region), str(dcl)))
