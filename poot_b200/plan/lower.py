"""Lowering of a compiled ``Program`` to the launch list the device executor walks.

``compile_graph`` decides, per equation, which kernel family runs it and which equations are absorbed into a
neighbour's launch.  ``lower(program)`` turns that into an ordered list of ``Launch`` records with everything a
launcher needs: the weights it reads (by canonical name - sibling contractions that were merged into one GEMM name
all their weights, in row order), the epilogue, the values it consumes and the value whose bytes it produces, and the
width of that value's rows on the device.  Values that are views of another value resolve to the owner of the bytes.
A ``LaunchProgram`` also carries the arena layout: lifetime colouring of the produced values over the launch order
(the interval placement of ``plan/buffers.py``), in device bytes per token row, so the executor scales it by the engine's row capacity.

This is the counterpart of the reference's ``Program`` -> executor hand-off (crates/poot-graph-plan/src/compile.rs:923-1210:
plans, buffer plan and entry arena; crates/poot-executor/src/engine.rs:2454-2700: the walk that records the launches).
A launch list is a function of the model configuration only, not of the step's row count: the row-count dependent
choices (skinny or tiled GEMM, per-row or tensor-core attention, split-K) are made by the launchers at run time.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..ir.graph import Graph
from .compile import Program
from .refusal import Refusal

_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")


class LoweringRefused(ValueError):
    """The planned graph holds a dispatch this lowering has no launcher for; the caller keeps its own program."""


@dataclass
class Launch:
    op: str                        # embed | rmsnorm | gemm | rope_kv | attention | moe | rows
    eqn: int                       # equation of the planned graph that dispatches
    layer: int                     # model layer, -1 outside the layer stack
    out: int                       # value whose bytes this launch produces (owner)
    width: int                     # columns of a row of ``out`` on the device
    x: Optional[int] = None        # activation operand (owner value)
    resid: Optional[int] = None    # residual operand of a GEMM with the residual epilogue
    weights: Tuple[str, ...] = ()  # canonical weight names read (merged siblings in row order)
    bias: Tuple[str, ...] = ()     # canonical bias names added to the GEMM's rows
    epi: str = "store"             # store | swiglu | resid | f32
    dtype_bytes: int = 2           # device bytes per element of ``out``
    covers: Tuple[int, ...] = ()   # other dispatching equations this launch runs as well


@dataclass
class LaunchProgram:
    launches: List[Launch]
    row_bytes: Dict[int, Tuple[int, int]] = field(default_factory=dict)   # owner value -> (offset, bytes) per token row
    arena_row_bytes: int = 0           # arena bytes per token row after lifetime colouring
    sum_row_bytes: int = 0             # what separate buffers would take
    census: Dict[str, int] = field(default_factory=dict)


def _weight(g: Graph, by_value, v: int) -> Optional[str]:
    i = by_value.get(v)
    return i.name if i is not None and i.storage == "const" else None


def lower(program: Program) -> LaunchProgram:
    g, plans = program.graph, program.plans
    by_value = {i.value: i for i in g.inputs}
    prod = g.producers()
    users = g.users()
    out_names = {o.value: o.name for o in g.outputs}

    def owner(v: int) -> int:
        """The value whose bytes ``v`` reads: follow views, movement handled by the consumer, and merged siblings."""
        seen = 0
        while v in prod and seen < 64:
            k = prod[v]
            e, p = g.eqns[k], plans[k]
            if p.kind in ("view", "alias") and e.inputs:
                v = e.inputs[0]
            elif p.kind == "none" and e.op in ("reshape", "transpose", "slice", "broadcast", "cast") and e.inputs:
                v = e.inputs[0]
            elif p.kind == "none" and e.op == "fused_row" and (p.note or "").startswith("the per-head q / k norm"):
                v = e.inputs[0]
            elif k in merged_into:
                v = g.eqns[merged_into[k]].outputs[0]
                break
            else:
                break
            seen += 1
        return v

    def layer_of(names) -> int:
        for n in names:
            m = _LAYER.match(n or "")
            if m:
                return int(m.group(1))
        return -1

    def cols(v: int) -> int:
        return g.types[v].shape[-1]

    # sibling contractions merged into the first one's GEMM
    merged_into: Dict[int, int] = {}
    for k, p in enumerate(plans):
        m = re.match(r"rows concatenated into the GEMM of eqn (\d+)", p.note or "")
        if p.kind == "none" and m:
            merged_into[k] = int(m.group(1))
    siblings: Dict[int, List[int]] = {}
    for k, first in merged_into.items():
        siblings.setdefault(first, []).append(k)

    launches: List[Launch] = []
    covered = set()
    moe_blocks = _moe_blocks(g, plans)
    for k, (e, p) in enumerate(zip(g.eqns, plans)):
        if p.kind != "dispatch" or k in covered:
            continue
        if k in moe_blocks:                      # router GEMM .. combine: one launcher runs the whole block
            blk = moe_blocks[k]
            covered.update(blk["eqns"])
            launches.append(Launch("moe", k, blk["layer"], blk["out"], cols(blk["out"]), x=owner(blk["x"]),
                                   resid=owner(blk["resid"]) if blk["resid"] is not None else None,
                                   weights=tuple(blk["weights"]), epi="resid", covers=tuple(sorted(blk["eqns"] - {k}))))
            continue
        kern = p.kernels[0]
        if e.op == "gather" and kern == "poot_embed_gather":
            launches.append(Launch("embed", k, -1, e.outputs[0], cols(e.outputs[0]), x=e.inputs[1],
                                   weights=(_weight(g, by_value, e.inputs[0]) or "embed",)))
        elif e.op == "fused_row" and e.attrs.get("kind") == "rmsnorm":
            w = [n for n in (_weight(g, by_value, v) for v in e.inputs) if n]
            src = e.inputs[0]
            if _through_slice(g, plans, prod, src):          # the logit rows are selected before the final norm
                rows_out = -(k + 1)                            # a synthetic value: the selected rows
                launches.append(Launch("rows", k, -1, rows_out, cols(src), x=owner(src)))
                launches.append(Launch("rmsnorm", k, layer_of(w), e.outputs[0], cols(e.outputs[0]), x=rows_out,
                                       weights=tuple(w)))
            else:
                launches.append(Launch("rmsnorm", k, layer_of(w), e.outputs[0], cols(e.outputs[0]), x=owner(src),
                                       weights=tuple(w)))
        elif e.op in ("dense_contraction", "packed_contraction", "contraction_epilogue", "matmul"):
            group = [k] + sorted(siblings.get(k, []))
            names, biases, width = [], [], 0
            resid = None
            for j in group:
                ej = g.eqns[j]
                wn = [n for n in (_weight(g, by_value, v) for v in ej.inputs) if n]
                names.append(wn[0])
                width += cols(ej.outputs[0])
                if ej.op == "contraction_epilogue":
                    extra = ej.inputs[2] if len(ej.inputs) > 2 else None
                    bn = _bias_name(g, by_value, prod, extra) if extra is not None else None
                    if bn is not None:
                        biases.append(bn)
                    elif extra is not None:
                        resid = owner(extra)
            acts = [v for v in e.inputs if _weight(g, by_value, v) is None]
            x = owner(acts[0])
            out, epi, nbytes = e.outputs[0], "store", 2
            sw = _swiglu_consumer(g, plans, users, [g.eqns[j].outputs[0] for j in group])
            if sw is not None:
                out, epi, width = sw, "swiglu", cols(sw)
            elif resid is not None:
                epi = "resid"
            elif out_names.get(out) == "logits":
                epi, nbytes = "f32", 4
            launches.append(Launch("gemm", k, layer_of(names), out, width, x=x, resid=resid, weights=tuple(names),
                                   bias=tuple(biases), epi=epi, dtype_bytes=nbytes))
        elif e.op == "rope":
            # the launch rotates q and k and writes K/V; the value it produces for later launches is the rotated query
            group = [k] + [j for j, pj in enumerate(plans)
                           if pj.kind == "none" and (pj.note or "") == f"same launch as the rotary of eqn {k}"]
            qk = next((j for j in group if _feeds(g, plans, users, g.eqns[j].outputs[0], "attention")), k)
            qv = g.eqns[qk].outputs[0]
            src = owner(g.eqns[qk].inputs[0])
            # a rotary over part of the head width still yields whole query rows: as wide as the query projection
            width = cols(src) if src in prod and g.eqns[prod[src]].op in ("dense_contraction", "packed_contraction",
                                                                          "contraction_epilogue", "matmul") \
                else cols(qv) * g.types[qv].shape[-2]
            launches.append(Launch("rope_kv", k, _layer_near(launches), qv, width, x=src))
        elif e.op == "attention":
            q = owner(e.inputs[3])
            o = g.types[e.outputs[0]]
            launches.append(Launch("attention", k, _layer_near(launches), e.outputs[0], o.shape[-1] * o.shape[-3], x=q))
        else:
            raise LoweringRefused(f"eqn {k} ({e.op}, {p.kernels}) has no launcher")
    lp = LaunchProgram(launches, census=program.census)
    _colour(lp)
    return lp


def _feeds(g: Graph, plans, users, v: int, op: str, depth: int = 0) -> bool:
    """Whether ``v`` reaches an equation ``op`` through views and movement only."""
    if depth > 8:
        return False
    for u in users.get(v, []):
        e = g.eqns[u]
        if e.op == op:
            return True
        if e.op in ("reshape", "transpose", "slice", "broadcast", "cast") and _feeds(g, plans, users, e.outputs[0], op, depth + 1):
            return True
    return False


def _layer_near(launches: List[Launch]) -> int:
    for l in reversed(launches):
        if l.layer >= 0:
            return l.layer
    return 0


def _through_slice(g: Graph, plans, prod, v: int) -> bool:
    seen = 0
    while v in prod and seen < 16:
        e = g.eqns[prod[v]]
        if e.op == "slice":
            return True
        if plans[prod[v]].kind in ("view", "alias") and e.inputs:
            v = e.inputs[0]
            seen += 1
            continue
        return False
    return False


def _bias_name(g: Graph, by_value, prod, v: int) -> Optional[str]:
    """``v`` is a bias row broadcast over the step's rows: the name of the constant it comes from, else None."""
    seen = 0
    while seen < 8:
        i = by_value.get(v)
        if i is not None:
            return i.name if i.storage == "const" and i.name.endswith("_bias") else None
        if v not in prod:
            return None
        e = g.eqns[prod[v]]
        if e.op not in ("broadcast", "reshape", "cast") or not e.inputs:
            return None
        v = e.inputs[0]
        seen += 1
    return None


def _swiglu_consumer(g: Graph, plans, users, outs: List[int]) -> Optional[int]:
    """The output value of the gated activation that runs in this GEMM group's epilogue, if there is one."""
    for v in outs:
        for u in users.get(v, []):
            e = g.eqns[u]
            if e.op == "fused" and e.attrs.get("kind") == "swiglu" and plans[u].kind == "none":
                return e.outputs[0]
    return None


def _moe_blocks(g: Graph, plans) -> Dict[int, dict]:
    """Routed-experts blocks of the plan, keyed by the equation of their router GEMM: the five launches between the
    router logits and the combine run from one launcher."""
    by_value = {i.value: i for i in g.inputs}
    prod = g.producers()
    users = g.users()
    blocks: Dict[int, dict] = {}
    disp = [k for k, p in enumerate(plans) if p.kind == "dispatch"]
    for idx, k in enumerate(disp):
        if not plans[k].kernels or plans[k].kernels[0] != "poot_moe_route":
            continue
        # the router GEMM is the dispatch just before, the grouped GEMMs and the combine follow
        router = disp[idx - 1]
        rw = [n for n in (_weight(g, by_value, v) for v in g.eqns[router].inputs) if n]
        if not rw or "router" not in rw[0]:
            continue
        tail = []
        for j in disp[idx + 1:]:
            tail.append(j)
            if plans[j].kernels in (["poot_moe_combine"], ["poot_moe_scatter_combine"]):
                break
        comb = tail[-1]
        out = g.eqns[comb].outputs[0]
        resid, final = None, out
        for u in users.get(out, []):              # the residual add the combine kernel performs
            eu = g.eqns[u]
            if plans[u].kind == "none" and (eu.op == "add" or eu.attrs.get("region") == "residual_add"):
                others = [v for v in eu.inputs if v != out]
                resid, final = (others[0] if others else None), eu.outputs[0]
        acts = [v for v in g.eqns[router].inputs if _weight(g, by_value, v) is None]
        m = _LAYER.match(rw[0])
        blocks[router] = dict(eqns={router, k, *tail}, layer=int(m.group(1)) if m else 0, x=acts[0], resid=resid,
                              out=final, weights=rw)
    return blocks


def _colour(lp: LaunchProgram) -> None:
    """Lifetime colouring of the produced values over the launch order, in bytes per token row.  A residual GEMM may
    write over its own residual operand (the epilogue reads and writes the same element), so the two share bytes when
    the operand dies there; everything else gets bytes that no live value holds."""
    last: Dict[int, int] = {}
    for n, l in enumerate(lp.launches):
        for v in (l.x, l.resid):
            if v is not None:
                last[v] = n
    end = len(lp.launches)
    if lp.launches:
        last[lp.launches[-1].out] = end
    from .buffers import first_fit
    placed: list = []
    for n, l in enumerate(lp.launches):
        size = (l.width * l.dtype_bytes + 15) // 16 * 16
        if l.op in ("gemm", "moe") and l.epi == "resid" and l.resid is not None and last.get(l.resid, -1) == n \
                and l.resid in lp.row_bytes and lp.row_bytes[l.resid][1] == size:
            lp.row_bytes[l.out] = lp.row_bytes[l.resid]        # in place over the residual stream
            for item in placed:
                if item[0] == lp.row_bytes[l.resid][0] and item[3] == n:
                    item[3] = last.get(l.out, n)
            continue
        got, _, placed = first_fit([(l.out, size, n, last.get(l.out, n))], placed)
        lp.row_bytes[l.out] = got[l.out]
    lp.arena_row_bytes = max((o + z for o, z, _, _ in placed), default=0)
    lp.sum_row_bytes = sum(z for _, z, _, _ in placed)
