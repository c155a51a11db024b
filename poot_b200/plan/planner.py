"""Per-equation plans: which hand-written kernel runs an equation, or that nothing runs at all.

A plan is ``dispatch`` (kernel launches), ``view`` (a reinterpretation of bytes already in place), ``alias`` (the
output is its input) or ``host`` (a computed constant prepared once at load)
(crates/poot-graph-plan/src/types.rs:725-756, src/planner.rs:1-7, src/planner/choice.rs:1-6).  Kernel names are the
launchers exported by the kernel library, so the plan of a traced step can be compared with the launches the
engine really makes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..ir.graph import Eqn, Graph
from ..tensor import DType
from .refusal import Refusal

TARGET = "sm_100a"
VIEW_OPS = {"reshape", "cast_noop"}


@dataclass
class Plan:
    kind: str                       # dispatch | view | alias | none
    kernels: List[str] = field(default_factory=list)
    note: str = ""


def _rows(g: Graph, v: int) -> int:
    s = g.types[v].shape
    n = 1
    for d in s[:-1]:
        n *= d
    return n


def contraction_kernel(m: int, packed: Optional[str] = None) -> List[str]:
    """Row-count dispatch of the projection kernels (the same thresholds as ``ops.cuda_ops.linear``)."""
    if packed is not None:
        return ["poot_quant_gemv"] if m <= 4 else ["poot_quant_dequant_bf16", "poot_gemm_bf16_tcgen05"]
    if m <= 128:
        return ["poot_gemm_skinny"]
    return ["poot_gemm_bf16_tcgen05"]


def plan_eqn(g: Graph, k: int, e: Eqn, world: int = 1) -> Plan:
    op = e.op
    dt = tuple(str(g.types[v].dtype) for v in e.inputs)
    if op in ("reshape",):
        return Plan("view")
    if op == "cast":
        return Plan("dispatch", ["poot_cast"], "fused into the consumer when it narrows on store")
    if op in ("transpose", "slice", "concat", "broadcast"):
        return Plan("dispatch", ["movement"], "standalone movement: only reached when no composite absorbed it")
    if op == "iota":
        return Plan("none", note="materialised by its consumer")
    if op == "gather":
        return Plan("dispatch", ["poot_embed_gather"])
    if op in ("dense_row_gather", "packed_row_gather"):
        return Plan("dispatch", ["poot_quant_row_gather" if op.startswith("packed") else "poot_embed_gather"])
    if op in ("scatter_update", "dynamic_update_slice"):
        return Plan("dispatch", ["poot_rope_kv_write"], "paged K/V write through the write map (-1 skips)")
    if op == "rope":
        return Plan("dispatch", ["poot_rope_kv_write"], "rotary + q/k norm + K/V write in one launch")
    if op == "attention":
        split = ["poot_attn_paged", "poot_attn_combine"] if _rows(g, e.outputs[0]) <= 256 else ["poot_attn_paged"]
        return Plan("dispatch", split, f"key={e.attrs.get('key')} n_rep={e.attrs.get('n_rep')}")
    if op == "fused_row" and e.attrs.get("kind") == "rmsnorm":
        return Plan("dispatch", ["poot_tp_norm" if world > 1 else "poot_rmsnorm"])
    if op == "fused_row" and e.attrs.get("kind") == "causal_conv_silu":
        return Plan("dispatch", ["poot_causal_conv_silu"], f"{e.attrs.get('taps')} taps, window carried per sequence")
    if op == "fused_row" and e.attrs.get("kind") == "gated_rmsnorm":
        return Plan("dispatch", ["poot_gated_rmsnorm"], f"gate {'before' if e.attrs.get('gate_first') else 'after'} the norm ({e.attrs.get('act')})")
    if op == "fused" and e.attrs.get("kind") == "swiglu":
        return Plan("none", note="runs in the gate/up contraction's epilogue (interleaved gate and up rows)")
    if op == "fused":
        return Plan("dispatch", ["poot_add"] if e.attrs.get("ops", 0) <= 2 else ["elementwise"])
    if op in ("dense_contraction", "matmul"):
        return Plan("dispatch", contraction_kernel(_rows(g, e.outputs[0])))
    if op == "packed_contraction":
        return Plan("dispatch", contraction_kernel(_rows(g, e.outputs[0]), e.attrs["format"]))
    if op == "contraction_epilogue":
        packed = e.attrs["head"] == "packed_contraction"
        return Plan("dispatch", contraction_kernel(_rows(g, e.outputs[0]), "packed" if packed else None),
                    "residual add in the epilogue")
    if op == "all_reduce":
        return Plan("none", note="fused into the producing contraction's epilogue (one-shot peer stores or reduce-scatter)")
    if op == "all_gather":
        return Plan("none", note="fused into the consuming contraction (peer push into the gather buffer)")
    if op == "sample_token":
        rule = e.attrs.get("rule", "greedy")
        return Plan("dispatch", ["poot_argmax"] if rule == "greedy" else ["poot_sample_gumbel"])
    if op == "random_uniform":
        return Plan("dispatch", ["poot_random_uniform"])
    if op == "arg_top_k":
        return Plan("dispatch", ["poot_moe_route"])
    if op in ("indexed_matmul", "grouped_dense_contraction", "expert_group"):
        return Plan("dispatch", ["poot_gemm_skinny_grouped"])
    if op in ("add", "sub", "mul", "div", "max", "neg", "exp", "tanh", "sqrt", "recip", "select", "ge", "and", "or",
              "xor", "log", "erf", "not", "geu", "remu", "shl", "shr", "clz", "reduce"):
        return Plan("dispatch", ["elementwise"], "unfused primitive")
    if op == "scan":
        # recurrences over a sequence's own state rows: the gated delta rule (D x D state per head) and the Mamba2
        # recurrence (N x P state per head); the state update and the output come out of one launch per layer
        kind = e.attrs.get("family")
        kernel = {"delta_rule": "poot_gdn_scan", "ssd": "poot_ssd_scan"}.get(kind)
        if kind == "delta_rule" and g.types[e.inputs[3]].shape[-1] > 1:
            kernel, kind = "poot_kda_scan", "delta_rule with a decay per key channel"
        if kernel is None:
            raise Refusal(k, op, dt, TARGET, f"no kernel for the {kind!r} recurrence")
        return Plan("dispatch", [kernel], f"{kind}: state carried per (sequence, head) in shared memory")
    if op == "ngram_hash":
        # wrapping 64-bit multiplies, xors and a remainder by a 32-bit prime per head: one thread per (token, head)
        return Plan("dispatch", ["poot_ngram_hash"], f"{len(e.attrs['primes'])} heads over a window of {g.types[e.inputs[0]].shape[0]}")
    if op == "block_top_k":
        # the exact radix select over each row's scores (ties at the cut: lowest position first)
        return Plan("dispatch", ["poot_index_select"], f"k={e.attrs.get('k')} of {g.types[e.inputs[0]].shape[-1]} candidates")
    if op in ("selected_attention", "packed_dequant", "all_to_all", "side_output"):
        raise Refusal(k, op, dt, TARGET, "no kernel family for this equation")
    raise Refusal(k, op, dt, TARGET, "unknown equation")


ABSORBING = {"attention", "rope", "scatter_update", "dynamic_update_slice", "dense_contraction", "packed_contraction",
             "contraction_epilogue", "matmul", "fused_row", "fused", "sample_token"}
MOVEMENT = {"transpose", "slice", "concat", "broadcast", "iota", "cast"}
CONTRACTIONS = {"dense_contraction", "packed_contraction", "contraction_epilogue"}


def plan_graph(g: Graph, world: int = 1) -> List[Plan]:
    """Plans of every equation, then the absorptions that make the plan match the launches of the device program:

    * contractions that read the same activations (q / k / v; gate / up) run as ONE GEMM over concatenated (or
      interleaved) weight rows: the first sibling dispatches, the others are ``none``;
    * the rotary of q and of k, the gathers of the rotary table rows and the K/V scatter are one ``rope_kv_write`` launch;
    * movement (transpose, slice, concat, broadcast, cast) whose consumers are kernels that index their operands
      themselves is a ``view``;
    * attention over a prefill piece (16 rows or more, head_dim 128, no soft cap) runs on the tensor-core flash kernel.
    """
    plans = [plan_eqn(g, k, e, world) for k, e in enumerate(g.eqns)]
    users = g.users()
    prod = g.producers()
    by_value = {i.value: i for i in g.inputs}
    outs = {o.value for o in g.outputs}

    def consumers(v, seen=None):
        """Non-movement equations that finally read ``v`` (looking through views and movement)."""
        seen = seen if seen is not None else set()
        res = []
        for u in users.get(v, []):
            e = g.eqns[u]
            if e.op in MOVEMENT or e.op == "reshape":
                if u not in seen:
                    seen.add(u)
                    res += consumers(e.outputs[0], seen)
            else:
                res.append(e.op)
        if v in outs:
            res.append("output")
        return res

    def bias_operand(e: Eqn) -> bool:
        """A ``residual_add`` epilogue whose extra operand is a bias row broadcast over the step's rows (not an
        activation): the contraction still merges with its siblings, the bias is added to the merged rows."""
        if e.op != "contraction_epilogue" or len(e.inputs) < 3:
            return False
        v, hops = e.inputs[2], 0
        while hops < 8:
            i = by_value.get(v)
            if i is not None:
                return i.storage == "const" and i.name.endswith("_bias")
            j = prod.get(v)
            if j is None or g.eqns[j].op not in ("broadcast", "reshape", "cast") or not g.eqns[j].inputs:
                return False
            v, hops = g.eqns[j].inputs[0], hops + 1
        return False

    first_by_input: Dict[int, int] = {}
    rope_seen: Dict[tuple, int] = {}
    for k, e in enumerate(g.eqns):
        if e.op == "fused_row" and e.attrs.get("kind") == "rmsnorm":
            names = [by_value[v].name for v in e.inputs if v in by_value and by_value[v].storage == "const"]
            if names and names[-1].endswith(("_q_norm", "_k_norm")) and set(consumers(e.outputs[0])) <= {"rope"}:
                plans[k] = Plan("none", note="the per-head q / k norm is evaluated inside rope_kv_write")
            continue
        if e.op in CONTRACTIONS and (e.attrs.get("region") != "residual_add" or bias_operand(e)):
            acts = [v for v in e.inputs if not (v in by_value and by_value[v].storage == "const")]
            x = acts[0] if acts else e.inputs[0]
            if x in first_by_input:
                plans[k] = Plan("none", note=f"rows concatenated into the GEMM of eqn {first_by_input[x]} (same activations)")
            else:
                first_by_input[x] = k
                if bias_operand(e):
                    plans[k] = Plan("dispatch", plans[k].kernels + ["poot_add"], "bias row added to the merged rows")
        elif e.op == "rope":
            # q and k of one layer come out of the same merged projection: one launch rotates both and writes K/V
            src, hops = e.inputs[0], 0
            while src in prod and hops < 16 and g.eqns[prod[src]].op not in CONTRACTIONS and g.eqns[prod[src]].inputs:
                src, hops = g.eqns[prod[src]].inputs[0], hops + 1
            j = prod.get(src)
            if j is not None and g.eqns[j].op in CONTRACTIONS:
                acts = [v for v in g.eqns[j].inputs if not (v in by_value and by_value[v].storage == "const")]
                key = ("proj", first_by_input.get(acts[0] if acts else g.eqns[j].inputs[0], j))
            else:
                key = ("rows",) + tuple(e.inputs[1:])
            if key in rope_seen:
                plans[k] = Plan("none", note=f"same launch as the rotary of eqn {rope_seen[key]}")
            else:
                rope_seen[key] = k
        elif e.op in ("scatter_update", "dynamic_update_slice"):
            plans[k] = Plan("none", note="K/V rows are written by rope_kv_write through the write map")
        elif e.op == "gather":
            t = by_value.get(e.inputs[0])
            if t is not None and t.computed and t.computed[0] in ("rope_cos", "rope_sin"):
                plans[k] = Plan("none", note="rotary table rows are read inside rope_kv_write")
            elif all(c in ABSORBING or c == "output" for c in consumers(e.outputs[0])) and \
                    any(c == "attention" for c in consumers(e.outputs[0])):
                plans[k] = Plan("none", note="paged K/V is read in place by the attention kernel")
        elif e.op in MOVEMENT:
            cs = consumers(e.outputs[0])
            if cs and all(c in ABSORBING or c == "output" for c in cs):
                plans[k] = Plan("view" if e.inputs else "none", note="layout handled by the consuming kernel")
        elif e.op == "fused" and e.attrs.get("kind") == "pointwise":
            cs = consumers(e.outputs[0])
            if cs and all(c == "attention" for c in cs):
                plans[k] = Plan("none", note="the mask is evaluated inside the attention kernel from positions")
        elif e.op == "attention":
            o = g.types[e.outputs[0]]
            rows, d = o.shape[-2], o.shape[-1]
            if rows >= 16 and d == 128 and not e.attrs.get("softcap"):
                plans[k] = Plan("dispatch", ["poot_attn_flash_prefill"], plans[k].note)
    _absorb_routed_experts(g, plans, users, prod)
    return plans


def _absorb_routed_experts(g: Graph, plans: List[Plan], users, prod) -> None:
    """A routed-experts block is five launches on the device: the router GEMM, ``moe_route`` (canonical scores, stable
    top-k, gates, the dense gate matrix), two grouped expert GEMMs (the activation is the first one's epilogue, the
    gate scaling the second one's) and ``moe_combine`` (which also adds into the residual stream).  Everything between
    the router logits and the weighted sum - score canonicalisation, ranks, masks, the softmax over the selected
    logits, gate gathers, the row broadcast, the activation - is evaluated inside those kernels, so those equations
    are ``none`` here.  Literal broadcasts shared by the blocks of several layers are absorbed once every user of
    theirs is inside some block."""
    blocks = []
    for k, e in enumerate(g.eqns):
        if e.op != "arg_top_k":
            continue
        # forward slice from the selected ids up to the weighted sum over the k slots
        region, frontier, end = set(), [k], None
        while frontier:
            i = frontier.pop()
            for v in g.eqns[i].outputs:
                for u in users.get(v, []):
                    if u in region:
                        continue
                    region.add(u)
                    ue = g.eqns[u]
                    if ue.op == "reduce" and any(g.eqns[prod[x]].op == "transpose" for x in ue.inputs if x in prod) and \
                            any(r in region and g.eqns[r].op == "indexed_matmul" for r in range(u)):
                        end = u if end is None else min(end, u)
                        continue
                    frontier.append(u)
        if end is None:
            continue
        region = {i for i in region if i <= end}
        anc, frontier = set(), [end, k] + sorted(region)
        while frontier:                                  # every ancestor up to the router GEMM / the block's input
            i = frontier.pop()
            for v in g.eqns[i].inputs:
                j = prod.get(v)
                if j is None or j in anc or j in region:
                    continue
                if g.eqns[j].op in CONTRACTIONS or g.eqns[j].op in ("matmul", "fused_row", "attention", "add"):
                    continue
                anc.add(j)
                frontier.append(j)
        blocks.append((k, end, region, anc))
    if not blocks:
        return
    fixed = set().union(*[r | {end, k} for k, end, r, _ in blocks])
    back = set().union(*[a for _, _, _, a in blocks]) - fixed
    changed = True
    while changed:                                       # keep the ancestors whose every use stays inside some block
        changed = False
        inside = fixed | back
        for j in list(back):
            if not all(u in inside for o in g.eqns[j].outputs for u in users.get(o, [])):
                back.discard(j)
                changed = True
    for k, end, region, anc in blocks:
        grouped = 0
        # few (token, slot) rows: one group per row reads only the selected experts.  More rows than experts: the rows
        # are grouped by expert on the device first (align + gather), and the combine scatters back per token.
        sel = g.types[g.eqns[k].inputs[0]]
        rows_k = (sel.numel // sel.shape[-1]) * g.eqns[k].attrs.get("k", 1)
        by_rows = rows_k > sel.shape[-1]
        if by_rows:
            plans[k] = Plan("dispatch", ["poot_moe_route", "poot_moe_align", "poot_moe_gather_rows"],
                            "routing, block-aligned grouping of the rows by expert, gather into the grouped order")
        for i in sorted(region | (anc & back)):
            op = g.eqns[i].op
            if i == end:
                plans[i] = Plan("dispatch", ["poot_moe_scatter_combine" if by_rows else "poot_moe_combine"],
                                "sum of the gate-scaled expert outputs into the residual stream")
            elif op == "indexed_matmul":
                grouped += 1
                note = "SwiGLU in the epilogue" if grouped == 1 else "gate scaling in the epilogue"
                # tiles of 128 grouped rows (an average expert has more than 64 rows) go through the tiled tcgen05 kernel
                tiled = by_rows and rows_k // sel.shape[-1] > 64
                plans[i] = Plan("dispatch", ["poot_gemm_grouped_tiled" if tiled else "poot_gemm_skinny_grouped"], note)
            elif i != k:
                plans[i] = Plan("none", note=f"evaluated inside the routed-experts kernels (route of eqn {k})")
        for u in users.get(g.eqns[end].outputs[0], []):  # the residual add is moe_combine's accumulate
            if g.eqns[u].op == "add" or g.eqns[u].attrs.get("region") == "residual_add":
                plans[u] = Plan("none", note="the combine kernel adds into the residual stream")


def launch_census(plans: List[Plan]) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for p in plans:
        if p.kind == "dispatch":
            for kname in p.kernels:
                out[kname] = out.get(kname, 0) + 1
    return out
