"""Compiler feedback on the kernel library: registers, spills and shared memory per kernel entry, an occupancy model
of one sm_100 SM over those figures, and the choice among the instantiations of a kernel family.

The reference compiles candidate kernels through the device's JIT, reads back registers and local memory and takes the
cheapest candidate that does not spill (crates/poot-graph-plan/src/register_feedback.rs:1-8; the probe is
crates/poot-ptx-runtime/src/context.rs: ``cuFuncGetAttribute``).  Here the library is compiled ahead of time, so the
verdicts come from the offline assembler: the build runs ``ptxas -v`` over every translation unit and writes one row per
entry to ``lib/kernel_resources.json`` (``build.py::write_resource_table``).  ``ResourceTable`` answers three questions
without a device:

* ``verdict(entry)``: what one instantiation costs and how many CTAs of it one SM holds;
* ``choose(candidates)``: among instantiations that do the same work, the cheapest one that does not spill - or, when
  all spill, the one that moves the fewest spill bytes, with that stated in the verdict;
* ``spilling()``: every entry with local-memory traffic, which a test holds against the list of accepted ones so that
  a change that makes a hot kernel spill is seen at build time.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

# one sm_100 SM
REGISTERS_PER_SM = 65536
MAX_THREADS_PER_SM = 2048
MAX_CTAS_PER_SM = 32
SMEM_PER_SM = 228 * 1024
SMEM_PER_CTA = 227 * 1024
SMEM_CTA_RESERVE = 1024             # what the system keeps per resident CTA
REG_ALLOC_UNIT = 8                  # registers per thread are granted in eights
WARP_ALLOC_UNIT = 4                 # warps are granted per scheduler quad

_NAME = re.compile(r"(?:void\s+)?(?:[\w:]+::)?(\w+)\s*(<[^(]*>)?\s*\(")


@dataclass(frozen=True)
class Verdict:
    entry: str                      # mangled entry name
    kernel: str                     # plain kernel name, e.g. ``attn_paged_kernel``
    template: str                   # template arguments as written by the demangler, e.g. ``<128, 4>``
    source: str
    registers: int
    static_smem: int
    stack: int
    spill_stores: int
    spill_loads: int
    barriers: int

    @property
    def spills(self) -> bool:
        return bool(self.spill_stores or self.spill_loads)

    @property
    def spill_bytes(self) -> int:
        return self.spill_stores + self.spill_loads

    def resident_ctas(self, threads: int, dynamic_smem: int = 0) -> int:
        """CTAs of ``threads`` threads one SM holds at once: the smallest of the thread, register, shared-memory and
        CTA-slot limits.  0: the launch does not fit at all."""
        if threads <= 0 or threads > 1024:
            return 0
        warps = -(-threads // 32)
        warps_alloc = -(-warps // WARP_ALLOC_UNIT) * WARP_ALLOC_UNIT
        regs = -(-max(self.registers, 1) // REG_ALLOC_UNIT) * REG_ALLOC_UNIT
        per_cta_regs = regs * 32 * warps_alloc
        smem = self.static_smem + dynamic_smem
        if smem > SMEM_PER_CTA or per_cta_regs > REGISTERS_PER_SM:
            return 0
        by_threads = MAX_THREADS_PER_SM // (warps * 32)
        by_regs = REGISTERS_PER_SM // per_cta_regs
        by_smem = SMEM_PER_SM // (smem + SMEM_CTA_RESERVE)
        return max(0, min(by_threads, by_regs, by_smem, MAX_CTAS_PER_SM))

    def occupancy(self, threads: int, dynamic_smem: int = 0) -> float:
        """Resident warps over the SM's 64."""
        return self.resident_ctas(threads, dynamic_smem) * -(-threads // 32) / (MAX_THREADS_PER_SM // 32)


@dataclass(frozen=True)
class Choice:
    verdict: Verdict
    reason: str
    rejected: tuple                 # ((entry, why), ...)


class ResourceTable:
    def __init__(self, rows: Iterable[dict]):
        self.by_entry: Dict[str, Verdict] = {}
        self.by_kernel: Dict[str, List[Verdict]] = {}
        for r in rows:
            m = _NAME.search(r.get("signature", "")) if r.get("signature") != r["entry"] else None
            kernel, template = (m.group(1), (m.group(2) or "").replace(" ", "")) if m else (r["entry"], "")
            v = Verdict(r["entry"], kernel, template, r.get("source", ""), int(r["registers"]), int(r.get("static_smem", 0)),
                        int(r.get("stack", 0)), int(r.get("spill_stores", 0)), int(r.get("spill_loads", 0)), int(r.get("barriers", 0)))
            self.by_entry[v.entry] = v
            self.by_kernel.setdefault(kernel, []).append(v)

    @classmethod
    def load(cls, path: Optional[str] = None) -> "ResourceTable":
        p = Path(path) if path else Path(__file__).resolve().parent.parent / "lib" / "kernel_resources.json"
        if not p.exists() and path is None:               # the table is a product of the kernel build
            from ..build import build_kernels
            build_kernels()
        if not p.exists():
            raise FileNotFoundError(f"{p.name} is written by the kernel build (python -m poot_b200.build)")
        return cls(json.loads(p.read_text())["kernels"])

    def verdict(self, entry: str) -> Verdict:
        return self.by_entry[entry]

    def instantiations(self, kernel: str, template: Optional[str] = None) -> List[Verdict]:
        """Every compiled instantiation of ``kernel``; ``template`` narrows to one (spaces ignored)."""
        vs = self.by_kernel.get(kernel, [])
        if template is not None:
            t = template.replace(" ", "")
            vs = [v for v in vs if v.template == t]
        return list(vs)

    def spilling(self) -> List[Verdict]:
        return sorted((v for v in self.by_entry.values() if v.spills), key=lambda v: (v.kernel, v.template))

    def choose(self, candidates: Sequence[Verdict], threads: int, dynamic_smem: int = 0, cost=None) -> Choice:
        """The cheapest candidate that fits and does not spill.  ``cost(v)``: lower is better; by default the one that
        keeps the most warps resident, then the fewest registers.  When every fitting candidate spills the one with
        the fewest spill bytes is taken and the reason says so; when none fits, ``ValueError``."""
        if cost is None:
            cost = lambda v: (-v.occupancy(threads, dynamic_smem), v.registers)
        fits, rejected = [], []
        for v in candidates:
            if v.resident_ctas(threads, dynamic_smem) == 0:
                rejected.append((v.entry, f"{threads} threads with {v.registers} registers and {v.static_smem + dynamic_smem} B shared memory do not fit one SM"))
            else:
                fits.append(v)
        if not fits:
            raise ValueError("no candidate fits one SM: " + "; ".join(w for _, w in rejected))
        clean = [v for v in fits if not v.spills]
        if clean:
            rejected += [(v.entry, f"spills {v.spill_bytes} B per thread") for v in fits if v.spills]
            best = min(clean, key=cost)
            rejected += [(v.entry, "costs more") for v in clean if v is not best]
            return Choice(best, "cheapest candidate without spills", tuple(rejected))
        best = min(fits, key=lambda v: (v.spill_bytes, cost(v)))
        rejected += [(v.entry, f"spills {v.spill_bytes} B per thread") for v in fits if v is not best]
        return Choice(best, f"every candidate spills; this one moves the fewest bytes ({best.spill_bytes} B per thread)", tuple(rejected))


# planner kernel name -> library entry, where stripping ``poot_`` and adding ``_kernel`` does not give it
ENTRY_OF = {"poot_rope_kv_write": "rope_kv_kernel", "poot_gemm_skinny_grouped": "gemm_skinny_kernel", "poot_gemm_grouped_tiled": "gemm_bf16_tcgen05_kernel",
            "poot_quant_gemv": "quant_gemv_kernel", "poot_quant_row_gather": "quant_row_gather_kernel", "poot_tp_norm": "tp_norm_kernel",
            "poot_index_select": "index_select_kernel", "poot_planar_gemv": "planar_gemv_rows_kernel", "poot_cast": "cast_f32_bf16_kernel"}


def plan_resources(program, table: Optional[ResourceTable] = None) -> Dict[str, dict]:
    """The kernel choice record of a compiled program: for every kernel its plans dispatch, the library entry behind it,
    how many instantiations were built, the most registers any of them takes and the ones that spill
    (crates/poot-graph-plan/src/planner/choice.rs: the reference records ``Generated | Imported | NoDispatch`` beside
    each plan; every kernel here is a built one, so the record is what the build says about it).  A planner name with no
    entry in the library (``movement``, ``elementwise``: done by the consumer or by a library copy) maps to ``None``."""
    table = table or ResourceTable.load()
    out: Dict[str, dict] = {}
    for name, launches in sorted(program.census.items()):
        entry = ENTRY_OF.get(name, (name[len("poot_"):] if name.startswith("poot_") else name) + "_kernel")
        vs = table.instantiations(entry)
        if not vs:
            out[name] = None
            continue
        out[name] = {"entry": entry, "launches": launches, "instantiations": len(vs), "max_registers": max(v.registers for v in vs),
                     "max_static_smem": max(v.static_smem for v in vs), "spilling": [v.template or v.entry for v in vs if v.spills]}
    return out
