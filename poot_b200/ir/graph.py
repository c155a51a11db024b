"""Flat, typed SSA graph of primitive tensor ops.

The role of the reference's graph IR (crates/poot-graph-ir/src/graph.rs:424-1960, src/op.rs:1116-1533,
src/types.rs:66-73): static shapes only; a graph is a list of equations over values; inputs carry a storage
class (device input, constant, computed constant, per-step slot, carried state); outputs carry a role (result,
witness, export, next state).  A tracer may emit the primitive ops only.  The planner introduces *composite*
equations (attention, rope, fused regions, packed contractions ...); every composite carries the sub-graph of
primitives that defines it, which the CPU oracle evaluates - one semantic definition for every kernel.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

from ..tensor import DType

# ----------------------------------------------------------------------------------------------------------------
# op vocabulary
# ----------------------------------------------------------------------------------------------------------------
UNARY = ("neg", "exp", "log", "sqrt", "recip", "tanh", "erf", "not", "clz")
BINARY = ("add", "sub", "mul", "div", "max", "ge", "geu", "remu", "and", "or", "xor", "shl", "shr")
PRIMITIVES = UNARY + BINARY + (
    "select", "reduce", "broadcast", "cast", "reshape", "transpose", "slice", "concat", "iota", "gather",
    "scatter_update", "matmul", "packed_dequant", "arg_top_k", "indexed_matmul", "dynamic_update_slice", "scan", "ngram_hash",
    "random_uniform", "sample_token", "all_reduce", "all_gather", "all_to_all")
COMPOSITES = ("packed_contraction", "packed_row_gather", "dense_contraction", "grouped_dense_contraction",
              "dense_row_gather", "contraction_epilogue", "expert_group", "fused", "fused_row", "side_output",
              "attention", "rope", "block_top_k", "selected_attention", "rmsnorm", "swiglu")

SLOTS = ("token", "activation", "pos", "mrope_position", "slot_map", "write_map", "owned")
STATE_ROLES = ("positional", "blocked", "recurrent", "handoff", "sampler")
OUTPUT_ROLES = ("result", "witness", "export", "state_next")


class GraphError(ValueError):
    """An ill-typed equation or a malformed graph."""


@dataclass(frozen=True)
class TensorType:
    shape: Tuple[int, ...]
    dtype: DType

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        return self.numel * self.dtype.size

    def __str__(self) -> str:
        return f"{self.dtype}[{','.join(map(str, self.shape))}]"


@dataclass
class Input:
    """A graph input and where its bytes come from."""
    value: int
    name: str
    storage: str = "device"          # device | const | computed | slot | state
    slot: Optional[str] = None       # one of SLOTS when storage == "slot"
    state_role: Optional[str] = None  # one of STATE_ROLES when storage == "state"
    state_axis: Optional[int] = None
    range: Optional[Tuple[int, int]] = None   # declared value range of an I32 slot (checked at bind)
    computed: Optional[Tuple[str, tuple]] = None  # (kind, params) of a computed constant, e.g. ("rope_cos", ...)


@dataclass
class Output:
    value: int
    name: str
    role: str = "result"
    state_of: Optional[str] = None   # name of the state input this output replaces (donation)


@dataclass
class Eqn:
    op: str
    inputs: List[int]
    outputs: List[int]
    attrs: Dict[str, Any] = field(default_factory=dict)
    body: Optional["Graph"] = None   # decomposition of a composite over its inputs (in order)

    @property
    def is_composite(self) -> bool:
        return self.op in COMPOSITES


class Graph:
    def __init__(self):
        self.types: Dict[int, TensorType] = {}
        self.names: Dict[int, str] = {}
        self.inputs: List[Input] = []
        self.eqns: List[Eqn] = []
        self.outputs: List[Output] = []
        self._next = 0

    # ---- construction -----------------------------------------------------------------------------------------
    def new_value(self, ty: TensorType, name: Optional[str] = None) -> int:
        v = self._next
        self._next += 1
        self.types[v] = ty
        if name:
            self.names[v] = name
        return v

    def add_input(self, name: str, ty: TensorType, **kw) -> int:
        if any(i.name == name for i in self.inputs):
            raise GraphError(f"duplicate input {name!r}")
        v = self.new_value(ty, name)
        self.inputs.append(Input(v, name, **kw))
        return v

    def add_eqn(self, op: str, inputs: Sequence[int], attrs: Optional[Dict[str, Any]] = None,
                body: Optional["Graph"] = None) -> List[int]:
        attrs = dict(attrs or {})
        if op not in PRIMITIVES and op not in COMPOSITES:
            raise GraphError(f"unknown op {op!r}")
        in_types = [self.types[i] for i in inputs]
        from .infer import infer
        out_types = infer(op, attrs, in_types, body)
        outs = [self.new_value(t) for t in out_types]
        self.eqns.append(Eqn(op, list(inputs), outs, attrs, body))
        return outs

    def add_output(self, value: int, name: str, role: str = "result", state_of: Optional[str] = None) -> None:
        if role not in OUTPUT_ROLES:
            raise GraphError(f"unknown output role {role!r}")
        self.outputs.append(Output(value, name, role, state_of))

    # ---- queries ----------------------------------------------------------------------------------------------
    def input_named(self, name: str) -> Input:
        for i in self.inputs:
            if i.name == name:
                return i
        raise KeyError(name)

    def producers(self) -> Dict[int, int]:
        """value id -> index of the equation that defines it."""
        return {o: k for k, e in enumerate(self.eqns) for o in e.outputs}

    def users(self) -> Dict[int, List[int]]:
        u: Dict[int, List[int]] = {}
        for k, e in enumerate(self.eqns):
            for i in e.inputs:
                u.setdefault(i, []).append(k)
        return u

    def validate(self) -> None:
        """Every operand is defined before use, every output exists, types re-infer to the recorded ones."""
        from .infer import infer
        defined = {i.value for i in self.inputs}
        for k, e in enumerate(self.eqns):
            for i in e.inputs:
                if i not in defined:
                    raise GraphError(f"eqn {k} ({e.op}) uses undefined value {i}")
            got = infer(e.op, e.attrs, [self.types[i] for i in e.inputs], e.body)
            want = [self.types[o] for o in e.outputs]
            if got != want:
                raise GraphError(f"eqn {k} ({e.op}) infers {got}, recorded {want}")
            defined.update(e.outputs)
        for o in self.outputs:
            if o.value not in defined:
                raise GraphError(f"output {o.name!r} is undefined")

    def digest(self) -> str:
        """Stable structural digest (plan-summary tests pin it)."""
        h = hashlib.sha256()
        for i in self.inputs:
            h.update(f"in {i.name} {self.types[i.value]} {i.storage} {i.slot} {i.state_role}\n".encode())
        for e in self.eqns:
            attrs = sorted((k, repr(v)) for k, v in e.attrs.items())
            h.update(f"{e.op} {e.inputs} -> {e.outputs} {attrs} {e.body.digest() if e.body else ''}\n".encode())
        for o in self.outputs:
            h.update(f"out {o.name} {o.value} {o.role}\n".encode())
        return h.hexdigest()[:16]

    def summary(self) -> Dict[str, int]:
        counts: Dict[str, int] = {}
        for e in self.eqns:
            counts[e.op] = counts.get(e.op, 0) + 1
        return counts

    def copy(self) -> "Graph":
        g = Graph()
        g.types, g.names = dict(self.types), dict(self.names)
        g.inputs = [Input(**vars(i)) for i in self.inputs]
        g.eqns = [Eqn(e.op, list(e.inputs), list(e.outputs), dict(e.attrs), e.body) for e in self.eqns]
        g.outputs = [Output(**vars(o)) for o in self.outputs]
        g._next = self._next
        return g

    def __repr__(self) -> str:
        lines = [f"graph({len(self.inputs)} inputs, {len(self.eqns)} eqns, {len(self.outputs)} outputs)"]
        for i in self.inputs:
            lines.append(f"  %{i.value}: {self.types[i.value]} = {i.storage} {i.name}")
        for e in self.eqns:
            outs = ", ".join(f"%{o}: {self.types[o]}" for o in e.outputs)
            ins = ", ".join(f"%{i}" for i in e.inputs)
            lines.append(f"  {outs} = {e.op}({ins}) {e.attrs if e.attrs else ''}")
        for o in self.outputs:
            lines.append(f"  -> {o.role} {o.name} = %{o.value}")
        return "\n".join(lines)
