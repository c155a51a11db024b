"""``python -m benchmarks.harness <command>``

    run      --model random:llama-3-8b --scenario decode-curve --isl 128 2048 --osl 128 --repeats 5 --out results/<id>
             one row per (isl, repeat) appended to <out>/results.jsonl, each behind the host-load meter
    validate <run dir>...                 every row against the contract; exit 1 on the first set with a bad row
    compare  --baseline <dir>... --candidate <dir>...   one verdict per cell; exit 0 / 1 (worse or broken) / 2 (unverified)
    report   <run dir>...                 medians with ranges per cell
    quiet                                 wait until the host is quiet (exit 1 if it never is)
"""
from __future__ import annotations

import argparse
import statistics
import sys

from . import contract, hostload, runner, verdicts


def cmd_run(a) -> int:
    bad = 0
    for isl in a.isl:
        for rep in range(1, a.repeats + 1):
            cell = lambda: runner.run_cell(a.model, a.scenario, isl, a.osl, rep, a.requests, a.rows, a.seed,
                                           a.storage_dtype, observer=runner.Observer())
            row = hostload.run_quiet(cell) if not a.no_host_meter else cell()
            runner.append_row(a.out, row)
            bad += row["status"] != "ok"
            print(f"isl={isl} repeat={rep}: {row['status']}"
                  + (f" decode {row['decode_tok_s']:.1f} tok/s ttft {row['ttft_ms']:.1f} ms" if row["status"] == "ok"
                     and row.get("decode_tok_s") else f" {row.get('reason', '')}"), flush=True)
    return 1 if bad else 0


def cmd_validate(a) -> int:
    rc = 0
    for d in a.runs:
        for i, row in enumerate(runner.load_rows(d)):
            for e in contract.row_errors(row):
                print(f"{d} row {i}: {e}")
                rc = 1
    return rc


def cmd_compare(a) -> int:
    ra = [r for d in a.baseline for r in runner.load_rows(d)]
    rb = [r for d in a.candidate for r in runner.load_rows(d)]
    cells = verdicts.compare_sets(ra, rb, verdicts.load_policy(a.policy))
    print(verdicts.render(cells))
    return verdicts.exit_code(cells)


def cmd_report(a) -> int:
    rows = [r for d in a.runs for r in runner.load_rows(d)]
    cells = {}
    for r in rows:
        cells.setdefault(contract.cell_key(r), []).append(r)
    print("| model | scenario | isl | osl | placement | storage | ok/total | decode tok/s (median, range) | ttft ms | "
          "peak VRAM GiB at inference |")
    print("|---|---|---|---|---|---|---|---|---|---|")
    for k, rs in sorted(cells.items(), key=lambda kv: tuple(str(p) for p in kv[0])):
        ok = [r for r in rs if r["status"] == "ok"]
        ds = [contract.derive_row(r) for r in ok]
        tok = [d["decode_tok_s"] for d in ds if d["decode_tok_s"]]
        tt = [d["ttft_ms"] for d in ds if d["ttft_ms"]]
        vr = [r["memory"]["inference_peak_vram_bytes"] for r in ok if (r.get("memory") or {}).get("inference_peak_vram_bytes")]
        f = lambda xs, s=1.0: "-" if not xs else f"{statistics.median(xs) * s:.4g} [{min(xs) * s:.4g}, {max(xs) * s:.4g}]"
        print("| " + " | ".join(str(p) for p in k) + f" | {len(ok)}/{len(rs)} | {f(tok)} | {f(tt)} | {f(vr, 2**-30)} |")
    return 0


def cmd_quiet(a) -> int:
    ok = hostload.wait_quiet(hostload.Meter())
    print("quiet" if ok else "the host never went quiet")
    return 0 if ok else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m benchmarks.harness", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run")
    r.add_argument("--model", required=True)
    r.add_argument("--scenario", default="decode-curve", choices=contract.SCENARIOS)
    r.add_argument("--isl", type=int, nargs="+", default=[128])
    r.add_argument("--osl", type=int, default=128)
    r.add_argument("--repeats", type=int, default=5)
    r.add_argument("--requests", type=int, default=1)
    r.add_argument("--rows", type=int, default=1)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--storage-dtype", default="bf16")
    r.add_argument("--no-host-meter", action="store_true")
    r.add_argument("--out", required=True)
    r.set_defaults(fn=cmd_run)
    v = sub.add_parser("validate")
    v.add_argument("runs", nargs="+")
    v.set_defaults(fn=cmd_validate)
    c = sub.add_parser("compare")
    c.add_argument("--baseline", nargs="+", required=True)
    c.add_argument("--candidate", nargs="+", required=True)
    c.add_argument("--policy", default=None)
    c.set_defaults(fn=cmd_compare)
    p = sub.add_parser("report")
    p.add_argument("runs", nargs="+")
    p.set_defaults(fn=cmd_report)
    q = sub.add_parser("quiet")
    q.set_defaults(fn=cmd_quiet)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
