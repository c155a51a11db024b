"""Tracer: model code is an ordinary Python function over ``Traced`` values that records a flat graph.

Counterpart of the reference's ``Builder`` / ``Traced`` / ``Outputs`` (crates/poot-graph-ir/src/builder.rs:752-2530).
Scalars are materialised as rank-0 constants; trace budgets (equation count) guard against runaway tracers
(``TraceLimits``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Union

import numpy as np

from ..tensor import DType
from .graph import Graph, GraphError, TensorType

Number = Union[int, float]


@dataclass
class TraceLimits:
    max_equations: int = 2_000_000
    max_value_bytes: int = 1 << 40


class TraceBudgetExceeded(GraphError):
    pass


class Traced:
    """A value being traced; arithmetic operators record equations on the owning builder."""
    __slots__ = ("b", "v")

    def __init__(self, builder: "Builder", value: int):
        self.b, self.v = builder, value

    @property
    def type(self) -> TensorType:
        return self.b.g.types[self.v]

    @property
    def shape(self):
        return self.type.shape

    @property
    def dtype(self) -> DType:
        return self.type.dtype

    def _other(self, o) -> "Traced":
        return o if isinstance(o, Traced) else self.b.scalar(o, self.dtype)

    def __add__(self, o): return self.b.binary("add", self, self._other(o))
    def __radd__(self, o): return self.b.binary("add", self._other(o), self)
    def __sub__(self, o): return self.b.binary("sub", self, self._other(o))
    def __rsub__(self, o): return self.b.binary("sub", self._other(o), self)
    def __mul__(self, o): return self.b.binary("mul", self, self._other(o))
    def __rmul__(self, o): return self.b.binary("mul", self._other(o), self)
    def __truediv__(self, o): return self.b.binary("div", self, self._other(o))
    def __rtruediv__(self, o): return self.b.binary("div", self._other(o), self)
    def __neg__(self): return self.b.unary("neg", self)
    def __matmul__(self, o): return self.b.matmul(self, o)

    def reshape(self, *shape): return self.b.reshape(self, shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape)
    def transpose(self, *perm): return self.b.transpose(self, perm[0] if len(perm) == 1 and isinstance(perm[0], (tuple, list)) else perm)
    def cast(self, dtype: DType): return self.b.cast(self, dtype)
    def sum(self, axis=-1, keepdim=False): return self.b.reduce(self, "sum", axis, keepdim)
    def max(self, axis=-1, keepdim=False): return self.b.reduce(self, "max", axis, keepdim)


class Builder:
    def __init__(self, limits: Optional[TraceLimits] = None):
        self.g = Graph()
        self.limits = limits or TraceLimits()
        self._scalars: Dict[Any, Traced] = {}

    # ---- inputs ---------------------------------------------------------------------------------------------
    def input(self, name: str, shape: Sequence[int], dtype: DType, **kw) -> Traced:
        return Traced(self, self.g.add_input(name, TensorType(tuple(shape), dtype), **kw))

    def slot(self, name: str, shape, dtype: DType, slot: str, range=None) -> Traced:
        return self.input(name, shape, dtype, storage="slot", slot=slot, range=range)

    def const(self, name: str, shape, dtype: DType) -> Traced:
        return self.input(name, shape, dtype, storage="const")

    def computed(self, name: str, shape, dtype: DType, kind: str, params: tuple) -> Traced:
        return self.input(name, shape, dtype, storage="computed", computed=(kind, params))

    def state(self, name: str, shape, dtype: DType, role: str, axis: Optional[int] = None) -> Traced:
        return self.input(name, shape, dtype, storage="state", state_role=role, state_axis=axis)

    def scalar(self, x: Number, dtype: DType) -> Traced:
        key = (float(x) if dtype.is_float else int(x), dtype)
        t = self._scalars.get(key)
        if t is None:
            name = f"lit.{dtype}.{len(self._scalars)}"
            t = self.input(name, (), dtype, storage="computed", computed=("literal", (key[0],)))
            self._scalars[key] = t
        return t

    # ---- emit -----------------------------------------------------------------------------------------------
    def emit(self, op: str, inputs: Sequence[Traced], attrs=None, body=None) -> List[Traced]:
        if len(self.g.eqns) >= self.limits.max_equations:
            raise TraceBudgetExceeded(f"trace exceeds {self.limits.max_equations} equations")
        outs = self.g.add_eqn(op, [t.v for t in inputs], attrs, body)
        return [Traced(self, o) for o in outs]

    def unary(self, op: str, x: Traced) -> Traced:
        return self.emit(op, [x])[0]

    def binary(self, op: str, a: Traced, b: Traced) -> Traced:
        return self.emit(op, [a, b])[0]

    def select(self, cond: Traced, t: Traced, f: Traced) -> Traced:
        return self.emit("select", [cond, t, f])[0]

    def reduce(self, x: Traced, kind: str, axis: int, keepdim: bool = False) -> Traced:
        return self.emit("reduce", [x], {"kind": kind, "axis": axis, "keepdim": keepdim})[0]

    def broadcast(self, x: Traced, shape) -> Traced:
        if tuple(shape) == tuple(x.shape):
            return x
        return self.emit("broadcast", [x], {"shape": tuple(shape)})[0]

    def cast(self, x: Traced, dtype: DType) -> Traced:
        if x.dtype == dtype:
            return x
        return self.emit("cast", [x], {"dtype": dtype})[0]

    def reshape(self, x: Traced, shape) -> Traced:
        shape = list(shape)
        if -1 in shape:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            shape[shape.index(-1)] = x.type.numel // known
        if tuple(shape) == tuple(x.shape):
            return x
        return self.emit("reshape", [x], {"shape": tuple(shape)})[0]

    def transpose(self, x: Traced, perm) -> Traced:
        perm = tuple(p % len(x.shape) for p in perm)
        if perm == tuple(range(len(perm))):
            return x
        return self.emit("transpose", [x], {"perm": perm})[0]

    def slice(self, x: Traced, axis: int, start: int, size: int) -> Traced:
        axis %= len(x.shape)
        starts = [0] * len(x.shape)
        sizes = list(x.shape)
        starts[axis], sizes[axis] = start, size
        return self.emit("slice", [x], {"starts": tuple(starts), "sizes": tuple(sizes)})[0]

    def concat(self, xs: Sequence[Traced], axis: int) -> Traced:
        if len(xs) == 1:
            return xs[0]
        return self.emit("concat", list(xs), {"axis": axis % len(xs[0].shape)})[0]

    def iota(self, shape, axis: int, dtype: DType = DType.I32) -> Traced:
        return self.emit("iota", [], {"shape": tuple(shape), "axis": axis % len(shape), "dtype": dtype})[0]

    def gather(self, x: Traced, idx: Traced, axis: int = 0) -> Traced:
        return self.emit("gather", [x, idx], {"axis": axis})[0]

    def scatter_update(self, x: Traced, idx: Traced, upd: Traced) -> Traced:
        """Rows ``idx`` of ``x`` replaced by ``upd`` (``idx == -1`` writes nothing; duplicates are refused at bind)."""
        return self.emit("scatter_update", [x, idx, upd])[0]

    def dynamic_update_slice(self, x: Traced, upd: Traced, start: Traced, axis: int) -> Traced:
        return self.emit("dynamic_update_slice", [x, upd, start], {"axis": axis % len(x.shape)})[0]

    def matmul(self, a: Traced, b: Traced, precision: str = "narrow") -> Traced:
        return self.emit("matmul", [a, b], {"precision": precision})[0]

    def indexed_matmul(self, x: Traced, w: Traced, idx: Traced, precision: str = "narrow") -> Traced:
        return self.emit("indexed_matmul", [x, w, idx], {"precision": precision})[0]

    def packed_dequant(self, packed: Traced, fmt: str, shape) -> Traced:
        return self.emit("packed_dequant", [packed], {"format": fmt, "shape": tuple(shape)})[0]

    def arg_top_k(self, rank: Traced, k: int) -> Traced:
        return self.emit("arg_top_k", [rank], {"k": k})[0]

    def scan(self, family: str, operands: Sequence[Traced], chunk: int = 64):
        """A bounded recurrence over the sequence axis with one packed result ``[1, H, L + S, W]``: rows ``..L`` are the
        sequence output, rows ``L..`` the carried state (crates/poot-graph-ir/src/op.rs:1427-1435, 3084-3216).
        ``delta_rule``: operands ``[q, k, v, g, beta, s_in]`` with q/k/v ``[1,H,L,D]``, g (log domain) ``[1,H,L,1]`` or,
        with a decay per key channel, ``[1,H,L,D]``, beta ``[1,H,L,1]``, ``s_in[1,H,D,D]``.  ``ssd``: ``[x, b, c, delta, a, d, h_in]`` with ``x[1,H,L,P]``, b/c
        ``[1,H,L,N]``, ``delta[1,H,L,1]``, a/d ``[1,H,1,1]``, ``h_in[1,H,N,P]``.  Returns ``(y, state_out)``."""
        first = operands[0]
        _, H, L, Wd = first.shape
        S = Wd if family == "delta_rule" else operands[1].shape[3]
        out = self.emit("scan", list(operands), {"family": family, "chunk": chunk, "shape": (1, H, L + S, Wd)})[0]
        return self.slice(out, 2, 0, L), self.slice(out, 2, L, S)

    def ngram_hash(self, window: Traced, context: int, multipliers, primes, offsets, heads_per_order: int, eos: int) -> Traced:
        """Hashed n-gram ids of a token run: ``window[context + t]`` I32 is the ``context`` tokens before the run followed
        by its ``t`` tokens; the result is ``[t, heads]`` I32 with ``heads = context * heads_per_order``.  For token
        ``i`` (window index ``context + i``) the order-2 mix is ``m0 * s0 ^ m1 * s1`` over wrapping 64-bit words
        (``s0`` the token, ``s1`` the one before it) and the order-3 mix xors ``m2 * s2``, where ``s2`` is the token two
        back, or ``eos`` when ``s1`` is ``eos`` (a context that ends a segment hides what precedes it).  Head ``h`` of
        order ``2 + h // heads_per_order`` is ``mix % primes[h] + offsets[h]`` (crates/poot-models/src/components/
        ple.rs ``row_ids``).  One equation: 64-bit integer arithmetic is native on the device."""
        return self.emit("ngram_hash", [window], {"context": int(context), "multipliers": tuple(int(m) for m in multipliers),
                                                   "primes": tuple(int(p) for p in primes), "offsets": tuple(int(o) for o in offsets),
                                                   "heads_per_order": int(heads_per_order), "eos": int(eos)})[0]

    def random_uniform(self, seed: Traced, cols: int) -> Traced:
        return self.emit("random_uniform", [seed], {"cols": cols})[0]

    def sample_token(self, rule: str, logits: Traced, noise=None, params=None, top_k=None) -> Traced:
        ins = [logits] + [t for t in (noise, params, top_k) if t is not None]
        return self.emit("sample_token", ins, {"rule": rule, "has_noise": noise is not None,
                                                "has_params": params is not None, "has_top_k": top_k is not None})[0]

    def all_reduce(self, x: Traced, op: str = "sum") -> Traced:
        return self.emit("all_reduce", [x], {"op": op})[0]

    def all_gather(self, x: Traced, axis: int, world: int) -> Traced:
        return self.emit("all_gather", [x], {"axis": axis % len(x.shape), "world": world})[0]

    # ---- outputs --------------------------------------------------------------------------------------------
    def output(self, x: Traced, name: str, role: str = "result", state_of: Optional[str] = None) -> None:
        self.g.add_output(x.v, name, role, state_of)

    def finish(self) -> Graph:
        self.g.validate()
        return self.g
