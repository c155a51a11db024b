"""``poot plan MODEL``: what the planner makes of one step of a checkpoint's model, without loading a weight.

Prints the pass log, the equations before and after, the launch census (kernel -> launches per step), the plan digest
(the value the committed digests pin), the numerics class the compiled graph implies with the tolerance that goes with
it, which carried states are updated in place and which are copied after the step, the bytes a step reads, and what
the kernel build reports for every dispatched kernel (the reference prints the same facts through its plan-digest and
launch-census recipes; crates/poot-graph-plan/src/compile.rs:923-1210)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List


def parse_plan(argv: List[str]) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="poot plan", description="compile one step of a model and print the plan")
    p.add_argument("model", help="checkpoint directory (config.json) or GGUF file")
    p.add_argument("--rows", type=int, default=1, help="sequences in the step")
    p.add_argument("--tokens", type=int, default=1, help="tokens per sequence (1: a decode step)")
    p.add_argument("--capacity", type=int, default=64, help="cache positions per sequence")
    p.add_argument("--world", type=int, default=1, help="tensor-parallel ranks")
    p.add_argument("--json", action="store_true", help="one JSON object instead of text")
    return p.parse_args(argv)


def plan_report(model, rows: int, tokens: int, capacity: int, world: int = 1) -> dict:
    from ..models.model import StepSpec
    from ..plan.compile import CompileOptions, compile_graph
    from ..plan.register_feedback import plan_resources
    spec = StepSpec(rows=rows, tokens=tokens, capacity=capacity, world=world) if world > 1 else StepSpec(rows=rows, tokens=tokens, capacity=capacity)
    g = model.trace(spec)
    prog = compile_graph(g, CompileOptions(world=world))
    commit = prog.state_commit
    try:
        resources = plan_resources(prog)
    except (FileNotFoundError, RuntimeError) as e:          # no compiler on this machine: the plan is still the plan
        resources = {"unavailable": str(e)}
    return {"family": model.cfg.family, "step": {"rows": rows, "tokens": tokens, "capacity": capacity, "world": world},
            "equations": {"traced": len(g.eqns), "planned": len(prog.graph.eqns)}, "digest": prog.graph.digest(),
            "passes": {k: v for k, v in prog.log.items() if k != "eqns_in"}, "dispatches": prog.dispatches, "census": dict(sorted(prog.census.items())),
            "numerics": {"class": prog.numerics, "tolerance": prog.tolerance}, "read_bytes": int(prog.read_traffic()),
            "state": {"in_place": sorted(commit.inplace.values()), "copied": [{"state": a, "reason": commit.reasons.get(a, "")} for a, _ in commit.copies]},
            "declines": [list(map(str, d)) for d in prog.declines][:32], "kernels": resources}


def main_plan(argv: List[str]) -> int:
    args = parse_plan(argv)
    from ..models.registry import Registry, UnsupportedFamily
    try:
        reg = Registry.builtin()
        if os.path.isdir(args.model):
            with open(os.path.join(args.model, "config.json")) as f:
                model = reg.resolve_hf(json.load(f))
        else:
            from ..load.gguf import read_index
            idx, _mm = read_index(args.model)
            model = reg.resolve_gguf(idx.metadata.get("general.architecture"), idx.metadata)
        rep = plan_report(model, args.rows, args.tokens, args.capacity, args.world)
    except (UnsupportedFamily, FileNotFoundError, ValueError, KeyError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    if args.json:
        print(json.dumps(rep, default=str))
        return 0
    s = rep["step"]
    print(f"{rep['family']}: {s['rows']} x {s['tokens']} tokens, capacity {s['capacity']}, world {s['world']}")
    print(f"equations {rep['equations']['traced']} -> {rep['equations']['planned']}   digest {rep['digest']}   dispatches {rep['dispatches']}   "
          f"reads {rep['read_bytes'] / 2**20:.1f} MiB per step")
    print(f"numerics {rep['numerics']['class']} (device vs oracle within {rep['numerics']['tolerance']:g})")
    print("passes: " + ", ".join(f"{k}={v}" for k, v in rep["passes"].items() if v not in (0, {}, None)))
    print("launches per step:")
    for k, n in rep["census"].items():
        r = rep["kernels"].get(k) if isinstance(rep["kernels"], dict) else None
        tail = f"   {r['entry']}: {r['instantiations']} built, <= {r['max_registers']} registers" + (f", spilling {r['spilling']}" if r["spilling"] else "") if r else ""
        print(f"  {n:4d}  {k}{tail}")
    print("state written in place: " + (", ".join(rep["state"]["in_place"]) or "none"))
    for c in rep["state"]["copied"]:
        print(f"state copied after the step: {c['state']} ({c['reason']})")
    if rep["declines"]:
        print(f"{len(rep['declines'])} declined rewrites, first: {' / '.join(rep['declines'][0])}")
    return 0
