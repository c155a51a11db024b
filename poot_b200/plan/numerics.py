"""Passes that decide numerics and limits: operand precision, narrow storage, range witnesses, legalization.

* ``select_operand_precision`` - the one pass that writes a non-exact operand precision.  The driver's policy is a
  permission, not an obligation: an op narrows its operands (to bf16, the fragment type of the target's matrix units)
  only where the planner runs it on a matrix unit; a schedule that gains nothing from rounding (the SIMT decode GEMV over
  a packed weight, a primitive the planner runs as plain elementwise work) stays exact, and an equation the tracer
  pinned exact (a router) stays exact under any policy (crates/poot-graph-plan/src/passes/operand_precision.rs:1-8).
* ``store_narrowed_activations`` - a value whose every reader narrows it to one dtype is stored narrow, rounded once by
  the kernel that computes it: the value is marked ``store`` = that dtype, which changes no result (the readers rounded
  it the same way) and halves the bytes the launch program's arena gives it (passes/narrow_storage.rs:1-8).
* ``check_narrow_ranges`` - the opt-in detector behind ``--check-ranges``: every activation a narrowed op rounds gets a
  validation witness (1 when an element would not round to a finite value) exported as a graph output of role
  ``witness`` whose name says which op, layer and operand left the range (passes/range_check.rs:1-8).
* ``legalize`` - device limits as a pass: a dense contraction whose weight exceeds what one buffer / one tensor map can
  address is split into row chunks that each fit, joined by a concat; what still does not fit is refused by name
  (passes/legalize.rs:1-8).  Tracers always emit the plain unsplit matmul.

Every pass is checked against the CPU oracle: the graph evaluates to the same values before and after (bit for bit,
except that a split contraction lets the host BLAS block its narrower chunks differently).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

from ..ir.graph import Eqn, Graph, Input, TensorType
from ..tensor import DType
from .refusal import Refusal

NARROWING = ("matmul", "dense_contraction", "packed_contraction", "contraction_epilogue", "indexed_matmul", "attention")
MATRIX_KERNELS = {"poot_gemm_skinny", "poot_gemm_bf16_tcgen05", "poot_gemm_skinny_grouped", "poot_gemm_grouped_tiled",
                  "poot_attn_flash_prefill"}
_LAYER = re.compile(r"layers\.(\d+)\.(\w+)")


@dataclass(frozen=True)
class Limits:
    """What one device buffer and one tensor map can hold (the B200 figures; tests pass smaller ones)."""
    max_buffer_bytes: int = 180 * 10**9
    max_tensor_rows: int = (1 << 31) - 1          # a tensor-map dimension and the kernels' 32-bit row indices
    max_elements: int = (1 << 40)                  # 64-bit element offsets throughout; a sanity bound


def select_operand_precision(g: Graph, policy: str = "narrow", world: int = 1) -> Dict[str, int]:
    """Write ``precision`` on every op that multiplies: ``exact``, or the policy where a matrix unit runs the op."""
    from .planner import plan_eqn
    if policy not in ("exact", "narrow", "split"):
        raise ValueError(f"matmul precision {policy!r}")
    out = {"exact": 0, policy: 0, "pinned": 0}
    for k, e in enumerate(g.eqns):
        if e.op not in NARROWING:
            continue
        if e.attrs.get("precision") == "exact" and e.attrs.get("precision_by") != "pass":
            out["pinned"] += 1                   # the tracer's own choice (a router's logits): kept
            continue
        prec = "exact"
        if policy != "exact":
            try:
                kernels = plan_eqn(g, k, e, world).kernels
            except Refusal:
                kernels = []
            if any(kn in MATRIX_KERNELS for kn in kernels) or e.op == "attention":
                prec = policy
        e.attrs["precision"] = prec
        e.attrs["precision_by"] = "pass"
        _write_body(e, prec)
        out[prec] += 1
    return out


def _write_body(e: Eqn, prec: str) -> None:
    """A composite is defined by its body: the products inside it round the way the composite does."""
    if e.body is None:
        return
    for inner in e.body.eqns:
        if inner.op in NARROWING:
            inner.attrs["precision"] = prec
        _write_body(inner, prec)


def store_narrowed_activations(g: Graph) -> int:
    """Mark the producer of every f32 value whose readers all narrow it: ``store`` = ``"bf16"``.  Returns the count."""
    users = g.users()
    prod = g.producers()
    outs = {o.value for o in g.outputs}
    by_value = {i.value for i in g.inputs}
    n = 0
    for v, us in users.items():
        if v in outs or v in by_value or v not in prod or g.types[v].dtype != DType.F32:
            continue
        if not us or not all(_reads_narrowed(g, g.eqns[u], v) for u in us):
            continue
        p = g.eqns[prod[v]]
        if p.op in ("reshape", "transpose", "slice", "broadcast", "concat"):      # movement stores nothing of its own
            continue
        if p.attrs.get("store") != "bf16":
            p.attrs["store"] = "bf16"
            n += 1
    return n


def _reads_narrowed(g: Graph, e: Eqn, v: int) -> bool:
    """Whether ``e`` reads ``v`` as an operand it rounds to the narrow type."""
    if e.op in ("reshape", "transpose"):          # looks through pure views to the real readers
        users = g.users().get(e.outputs[0], [])
        return bool(users) and all(_reads_narrowed(g, g.eqns[u], e.outputs[0]) for u in users)
    if e.op not in NARROWING or e.attrs.get("precision", "narrow") == "exact":
        return False
    if e.op == "contraction_epilogue":
        return v in e.inputs[:2]                  # the residual operand of the epilogue is read exactly
    if e.op == "attention":
        return v in (e.inputs[0], e.inputs[2], e.inputs[3]) if len(e.inputs) > 3 else v in e.inputs[:3]
    return True


def check_narrow_ranges(g: Graph) -> List[str]:
    """Add one witness output per activation operand that a narrowed op rounds: 1 when an element is not finite after
    rounding (bf16 has f32's exponent range, so that is an infinity or a NaN already present).  Returns the names."""
    from ..ir.builder import Builder  # noqa: F401  (the op vocabulary the witnesses use)
    by_value = {i.value: i for i in g.inputs}
    names: List[str] = []
    watched = set()
    for k, e in list(enumerate(g.eqns)):
        if e.op not in NARROWING or e.attrs.get("precision", "narrow") == "exact":
            continue
        layer, role = "-", e.op
        for v in e.inputs:
            i = by_value.get(v)
            m = _LAYER.match(i.name) if i is not None and i.storage == "const" else None
            if m:
                layer, role = m.group(1), m.group(2)
                break
        for pos, v in enumerate(e.inputs):
            i = by_value.get(v)
            if (i is not None and i.storage in ("const", "computed", "slot")) or v in watched:
                continue                         # weight ranges are known at bind; index inputs are not rounded
            if g.types[v].dtype != DType.F32:
                continue
            watched.add(v)
            names.append(f"narrow_range.{k}.l{layer}.{role}.operand{pos}")
    # append the witness equations after the whole program (they read values that stay live to the end anyway)
    for name, v in zip(names, list(watched_order(g, watched))):
        ty = g.types[v]
        (neg,) = g.add_eqn("neg", [v])
        (mag,) = g.add_eqn("max", [v, neg])
        (same,) = g.add_eqn("ge", [v, v])                     # false exactly for NaN
        (notnan,) = g.add_eqn("cast", [same], {"dtype": DType.F32})
        lim = _literal(g, 3.3895313892515355e38)               # the largest finite bf16
        (big,) = g.add_eqn("ge", [mag, g.add_eqn("broadcast", [lim], {"shape": ty.shape})[0]])
        (bigf,) = g.add_eqn("cast", [big], {"dtype": DType.F32})
        one = g.add_eqn("broadcast", [_literal(g, 1.0)], {"shape": ty.shape})[0]
        (nanf,) = g.add_eqn("sub", [one, notnan])
        (bad,) = g.add_eqn("max", [bigf, nanf])
        flat = g.add_eqn("reshape", [bad], {"shape": (ty.numel,)})[0]
        (w,) = g.add_eqn("reduce", [flat], {"kind": "max", "axis": -1, "keepdim": False})
        g.add_output(w, name, role="witness")
    return names


def watched_order(g: Graph, watched) -> List[int]:
    """The watched values in the order their names were made (first reading op first)."""
    by_value = {i.value: i for i in g.inputs}
    seen, out = set(), []
    for e in g.eqns:
        if e.op not in NARROWING or e.attrs.get("precision", "narrow") == "exact":
            continue
        for v in e.inputs:
            if v in watched and v not in seen:
                seen.add(v)
                out.append(v)
    return out


def _literal(g: Graph, value: float) -> int:
    name = f"lit.f32.range.{value!r}"
    for i in g.inputs:
        if i.name == name:
            return i.value
    return g.add_input(name, TensorType((), DType.F32), storage="computed", computed=("literal", (value,)))


def failed_witnesses(outputs: Dict[str, object]) -> List[str]:
    """Names of the witnesses of an evaluated graph that fired."""
    import numpy as np
    return [n for n, v in outputs.items() if n.startswith("narrow_range.") and float(np.asarray(v).max()) != 0.0]


class LegalizeRefused(ValueError):
    pass


def legalize(g: Graph, limits: Optional[Limits] = None) -> Dict[str, int]:
    """Split every dense contraction whose weight does not fit one buffer / one tensor map into row chunks that do.
    A chunk is declared as its own constant input ``name#r0:r1`` (computed kind ``rows`` naming the weight and its row
    range), so a caller binds inputs against what this pass produced.  Returns ``{weight name: chunks}``."""
    lim = limits or Limits()
    by_value = {i.value: i for i in g.inputs}
    split: Dict[str, int] = {}
    k = 0
    while k < len(g.eqns):
        e = g.eqns[k]
        if e.op != "dense_contraction":
            k += 1
            continue
        w = next((v for v in e.inputs if v in by_value and by_value[v].storage == "const"), None)
        if w is None:
            k += 1
            continue
        ty = g.types[w]
        rows, cols = ty.shape
        row_bytes = cols * ty.dtype.size
        if ty.nbytes <= lim.max_buffer_bytes and rows <= lim.max_tensor_rows and ty.numel <= lim.max_elements:
            k += 1
            continue
        per = min(lim.max_tensor_rows, lim.max_buffer_bytes // row_bytes, lim.max_elements // max(cols, 1))
        if per < 1:
            raise LegalizeRefused(f"{by_value[w].name}: one row of {row_bytes} bytes exceeds the device's buffer limit")
        x = next(v for v in e.inputs if v != w)
        name = by_value[w].name
        pieces = []
        new_eqns: List[Eqn] = []
        for r0 in range(0, rows, per):
            r1 = min(rows, r0 + per)
            cw = g.add_input(f"{name}#{r0}:{r1}", TensorType((r1 - r0, cols), ty.dtype), storage="const",
                             computed=("rows", (name, r0, r1)))
            by_value[cw] = g.inputs[-1]
            sub = Graph()
            a, b = sub.add_input("in0", g.types[cw]), sub.add_input("in1", g.types[x])
            # the body of a dense contraction: x @ transpose(W)
            (t,) = sub.add_eqn("transpose", [a], {"perm": (1, 0)})
            (y,) = sub.add_eqn("matmul", [b, t], {"precision": e.attrs.get("precision", "narrow")})
            sub.add_output(y, "out0")
            out_ty = TensorType(g.types[e.outputs[0]].shape[:-1] + (r1 - r0,), g.types[e.outputs[0]].dtype)
            ov = g.new_value(out_ty)
            new_eqns.append(Eqn("dense_contraction", [cw, x], [ov], dict(e.attrs), sub))
            pieces.append(ov)
        cat = Eqn("concat", pieces, [e.outputs[0]], {"axis": len(g.types[e.outputs[0]].shape) - 1})
        g.eqns[k:k + 1] = new_eqns + [cat]
        split[name] = len(pieces)
        k += len(new_eqns) + 1
    # a weight that no equation reads any more is no longer an input of the program
    used = {v for e in g.eqns for v in e.inputs} | {o.value for o in g.outputs}
    g.inputs = [i for i in g.inputs if i.value in used or i.storage != "const"]
    return split


def bind_legalized(inputs: Dict[str, object], g: Graph) -> Dict[str, object]:
    """Bind the row chunks ``legalize`` declared from the whole weights in ``inputs``."""
    out = dict(inputs)
    for i in g.inputs:
        if i.computed and i.computed[0] == "rows" and i.name not in out:
            name, r0, r1 = i.computed[1]
            out[i.name] = inputs[name][r0:r1]
    return out
