"""``compile_graph(graph, options) -> Program``: passes, per-equation plans, buffer plan, step statistics
(crates/poot-graph-plan/src/compile.rs:923-1210)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..ir.graph import Graph
from . import passes
from .buffers import BufferPlan, plan_buffers
from .planner import Plan, launch_census, plan_graph


@dataclass
class CompileOptions:
    world: int = 1
    fuse: bool = True
    attention: bool = True
    stop_after: Optional[str] = None       # name of the last pass to run (pass-soundness tests walk the pipeline)
    precision: Optional[str] = None        # exact | narrow | split: run select_operand_precision + store_narrowed_activations
    check_ranges: bool = False             # add the range witnesses of the narrowed operands (--check-ranges)
    limits: Optional[object] = None        # numerics.Limits: legalize against these device limits


@dataclass
class Program:
    graph: Graph
    plans: List[Plan]
    buffers: BufferPlan
    log: Dict[str, object] = field(default_factory=dict)
    declines: List[tuple] = field(default_factory=list)

    @property
    def numerics(self) -> str:
        """The strongest numerics property of the compiled graph (``ir/analysis.py::implied_numerics``)."""
        from ..ir.analysis import implied_numerics
        return implied_numerics(self.graph)

    @property
    def tolerance(self) -> float:
        """How closely a device result is expected to follow the oracle, relative to ``max(|oracle element|, 1)``."""
        from ..ir.analysis import TIER2_TOLERANCE
        return TIER2_TOLERANCE[self.numerics]

    @property
    def state_commit(self):
        """Which state updates may overwrite their buffer and which are copied after the step (``plan/state_commit.py``)."""
        from .state_commit import plan_state_commit
        return plan_state_commit(self.graph)

    @property
    def census(self) -> Dict[str, int]:
        return launch_census(self.plans)

    @property
    def dispatches(self) -> int:
        return sum(len(p.kernels) for p in self.plans if p.kind == "dispatch")

    def read_traffic(self) -> int:
        """Bytes of constants (weights) the step reads: the decode roofline numerator
        (crates/poot-graph-plan/src/staged/traffic.rs:18).  Gather-only tables count their gathered rows."""
        g = self.graph
        users = g.users()
        total = 0
        for i in g.inputs:
            if i.storage != "const":
                continue
            ops = {g.eqns[u].op for u in users.get(i.value, [])}
            ty = g.types[i.value]
            if ops and ops <= {"gather", "dense_row_gather", "packed_row_gather"}:
                rows = max(g.types[g.eqns[u].outputs[0]].shape[0] for u in users[i.value])
                total += rows * ty.nbytes // ty.shape[0]
            elif ops:
                total += ty.nbytes
        return total


PIPELINE = ["canonicalize", "cse", "rope_fusion", "flash_attention", "form_selection", "form_recurrent_blocks", "dce", "fold_iota",
            "recognize_packed", "fold_dense_contractions", "lower_nonlast_reduces", "fuse_contraction_epilogues", "fuse", "dce2"]


def run_passes(g: Graph, opt: CompileOptions, log: Dict[str, object], declines: list) -> Graph:
    g = g.copy()
    for name in PIPELINE:
        if name == "canonicalize":
            log[name] = passes.canonicalize(g)
        elif name == "cse":
            log[name] = passes.cse(g)
        elif name == "rope_fusion":
            log[name] = passes.rope_fusion(g, declines)
        elif name == "flash_attention":
            log[name] = passes.flash_attention(g, declines) if opt.attention else 0
        elif name == "form_selection":
            from .selection import form_selection
            log[name] = form_selection(g, declines)
        elif name == "form_recurrent_blocks":
            from .recurrent_forms import form_recurrent_blocks
            log[name] = form_recurrent_blocks(g, declines) if any(e.op == "scan" for e in g.eqns) else {}
        elif name in ("dce", "dce2"):
            log[name] = passes.dce(g)
        elif name == "fold_iota":
            from .prepare import fold_iota
            log[name] = fold_iota(g)
        elif name == "lower_nonlast_reduces":
            from .prepare import lower_nonlast_reduces
            log[name] = lower_nonlast_reduces(g)
        elif name == "recognize_packed":
            log[name] = passes.recognize_packed(g)
        elif name == "fold_dense_contractions":
            log[name] = passes.fold_dense_contractions(g)
        elif name == "fuse_contraction_epilogues":
            log[name] = passes.fuse_contraction_epilogues(g) if opt.fuse else 0
        elif name == "fuse":
            log[name] = passes.fuse(g, declines) if opt.fuse else {}
        g.validate()
        if opt.stop_after == name:
            break
    return g


def compile_graph(graph: Graph, options: Optional[CompileOptions] = None) -> Program:
    opt = options or CompileOptions()
    log: Dict[str, object] = {"eqns_in": len(graph.eqns)}
    declines: list = []
    g = run_passes(graph, opt, log, declines)
    if opt.stop_after is None:
        from . import numerics
        if opt.limits is not None:
            log["legalize"] = numerics.legalize(g, opt.limits)
        if opt.precision is not None:
            log["select_operand_precision"] = numerics.select_operand_precision(g, opt.precision, opt.world)
            log["store_narrowed_activations"] = numerics.store_narrowed_activations(g)
        if opt.check_ranges:
            log["check_narrow_ranges"] = len(numerics.check_narrow_ranges(g))
        g.validate()
    log["eqns_out"] = len(g.eqns)
    plans = plan_graph(g, opt.world)
    return Program(g, plans, plan_buffers(g, plans), log, declines)
