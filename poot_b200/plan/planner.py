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
    if op in ("scan", "block_top_k", "selected_attention", "packed_dequant", "all_to_all", "side_output"):
        raise Refusal(k, op, dt, TARGET, "no kernel family for this equation")
    raise Refusal(k, op, dt, TARGET, "unknown equation")


def plan_graph(g: Graph, world: int = 1) -> List[Plan]:
    return [plan_eqn(g, k, e, world) for k, e in enumerate(g.eqns)]


def launch_census(plans: List[Plan]) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for p in plans:
        if p.kind == "dispatch":
            for kname in p.kernels:
                out[kname] = out.get(kname, 0) + 1
    return out
