"""Noise-aware comparison of two result sets: one verdict per cell, never "faster" without a band.

Each side of a cell is the repeats of one build.  A metric's band is twice the larger side's noise, where a side's
noise is the range five normal samples of its robust spread would show (2.33 sigma, sigma from the interquartile
range so one wild repeat does not set it), narrowed by sqrt(min_trials / n).  A candidate median outside the band is
a regression or an improvement; inside it the verdict is "within noise" only when the band is narrow enough to rule
out a loss of the metric's practical threshold - otherwise the cell is unverified, which is not success.  Too few
repeats, identical repeats, a failed repeat, rows that state different workloads or mixed builds on one side each
have their own verdict.  The rule and the verdict names are the reference comparator's
(benchmarks/harness/performance_receipt.py "metric_verdict", benchmarks/harness/bench.py "compare_cells"); the policy
numbers live in ``benchmarks/policy.json`` and nowhere else.
"""
from __future__ import annotations

import json
import math
import statistics
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

from . import contract

REGRESSION, IMPROVEMENT, WITHIN_NOISE = "regression", "improvement", "within noise"
UNVERIFIED, INVALID, CANDIDATE_FAILED = "unverified", "invalid", "candidate failed"
REPEAT_FAILED, NO_BASELINE, NEW, NOT_RUN, INCOMPARABLE = "repeat failed", "no baseline", "new", "not run", "incomparable"
COMPARED = frozenset({REGRESSION, IMPROVEMENT, WITHIN_NOISE})
FAILING = frozenset({REGRESSION, INVALID, CANDIDATE_FAILED, REPEAT_FAILED, INCOMPARABLE})
_ORDER = (INVALID, INCOMPARABLE, CANDIDATE_FAILED, REPEAT_FAILED, REGRESSION, NO_BASELINE, NOT_RUN, UNVERIFIED,
          WITHIN_NOISE, IMPROVEMENT, NEW)
RANGE_OF_FIVE = 2.33        # expected range of five normal samples, in sigma
IQR_SIGMA = 1.349           # interquartile range of a normal distribution, in sigma
POLICY_FILE = Path(__file__).resolve().parents[1] / "policy.json"


def load_policy(path: Optional[str] = None) -> dict:
    p = json.loads(Path(path or POLICY_FILE).read_text())
    for name, m in p["metrics"].items():
        if m.get("direction") not in ("higher", "lower"):
            raise ValueError(f"policy metric {name}: direction must be 'higher' or 'lower'")
        if not (0 < m["max_uncertainty"] <= m["practical_threshold"]):
            raise ValueError(f"policy metric {name}: need 0 < max_uncertainty <= practical_threshold")
    if not (2 <= p["min_trials"] <= p["max_trials"]):
        raise ValueError("policy: need 2 <= min_trials <= max_trials")
    return p


def spread(samples: Sequence[float]) -> float:
    q = statistics.quantiles(samples, n=4, method="inclusive")
    return (q[2] - q[0]) / IQR_SIGMA


def side_noise(samples: Sequence[float], min_trials: int) -> float:
    return RANGE_OF_FIVE * spread(samples) * math.sqrt(min_trials / len(samples))


def _repeats_hint(band: float, limit: float, n: int, max_trials: int) -> str:
    if limit > 0:
        need = math.ceil(n * (band / limit) ** 2)
        if need <= max_trials:
            return f" (about {need} repeats per side would fit; have {n})"
    return f" ({max_trials} repeats per side would not fit: the spread is the limit, not the count)"


def judge_metric(a: Sequence[float], b: Sequence[float], policy: dict, metric: str, failed_a: int = 0,
                 failed_b: int = 0) -> dict:
    """Baseline samples ``a`` against candidate samples ``b`` (one value per repeat)."""
    tol = policy["metrics"][metric]
    r = {"metric": metric, "verdict": None, "note": "", "n_a": len(a), "n_b": len(b), "median_a": None,
         "median_b": None, "range_a": None, "range_b": None, "relative_band": None, "budget_exhausted": False}

    def done(v, note=""):
        r["verdict"], r["note"] = v, note
        return r

    ok = lambda xs: all(isinstance(x, (int, float)) and math.isfinite(x) for x in xs)
    if not ok(a) or not ok(b):
        return done(INVALID, "non-finite sample")
    if not a:
        return done(NO_BASELINE, "the baseline has no successful run of this cell")
    if not b:
        return done(CANDIDATE_FAILED, "no successful candidate run")
    r.update(median_a=statistics.median(a), median_b=statistics.median(b), range_a=max(a) - min(a),
             range_b=max(b) - min(b))
    if failed_a or failed_b:
        return done(REPEAT_FAILED, f"{failed_a} baseline and {failed_b} candidate repeats failed")
    lo, hi = policy["min_trials"], policy["max_trials"]
    if len(a) < lo or len(b) < lo:
        return done(UNVERIFIED, f"needs {lo} runs per side, have {len(a)} and {len(b)}")
    if not (r["range_a"] or r["range_b"]):
        return done(UNVERIFIED, "the runs of both sides are identical, so no noise was observed")
    band = 2 * max(side_noise(a, lo), side_noise(b, lo))
    if band == 0:
        return done(UNVERIFIED, "the middle half of the runs are identical: the robust spread sizes no band")
    loss = r["median_a"] - r["median_b"]
    if tol["direction"] == "lower":
        loss = -loss
    if loss > band:
        return done(REGRESSION)
    if -loss > band:
        return done(IMPROVEMENT)
    scale = abs(r["median_a"])
    n = min(len(a), len(b))
    r["budget_exhausted"] = n >= hi
    if scale == 0:
        return done(UNVERIFIED, "a zero baseline median has no relative band")
    r["relative_band"] = band / scale
    if band / scale > tol["max_uncertainty"]:
        return done(UNVERIFIED, f"band {band / scale:.2%} exceeds the tolerated uncertainty {tol['max_uncertainty']:.2%}"
                    + _repeats_hint(band, tol["max_uncertainty"] * scale, n, hi))
    if (max(loss, 0) + band) / scale >= tol["practical_threshold"]:
        return done(UNVERIFIED, f"a loss of {tol['practical_threshold']:.1%} cannot be excluded"
                    + _repeats_hint(band, tol["practical_threshold"] * scale - max(loss, 0), n, hi))
    return done(WITHIN_NOISE)


def worst(verdicts: Iterable[str]) -> str:
    vs = list(verdicts)
    return next(v for v in _ORDER if v in vs)


def _cells(rows: Iterable[dict]) -> Dict[tuple, List[dict]]:
    out: Dict[tuple, List[dict]] = {}
    for r in rows:
        out.setdefault(contract.cell_key(r), []).append(r)
    return out


def _metrics_for(row: dict, policy: dict) -> List[str]:
    ms = [policy["headline_metric"]]
    if row.get("scenario") == "decode-curve":
        ms += policy["curve_point_metrics"]
    if row.get("scenario") == "prefill-1k":
        ms = ["prefill_tok_s", "ttft_ms"]
    return ms


def compare_cell(key, rows_a: Optional[List[dict]], rows_b: Optional[List[dict]], policy: dict) -> dict:
    cell = {"key": key, "verdict": None, "note": "", "entries": []}

    def done(v, note=""):
        cell["verdict"], cell["note"] = v, note
        return cell

    if rows_b is None:
        return done(NOT_RUN, "cell is not in the candidate")
    if rows_a is None:
        return done(NEW, "cell is not in the baseline")
    ok_a = [r for r in rows_a if r.get("status") == "ok"]
    ok_b = [r for r in rows_b if r.get("status") == "ok"]
    for side, rows in (("baseline", ok_a), ("candidate", ok_b)):
        bad = [e for r in rows for e in contract.row_errors(r)]
        if bad:
            return done(INVALID, f"the {side} has a row outside the contract: {bad[0]}")
        if len({r.get("build_sha") for r in rows}) > 1 or len({json.dumps(r.get("library_sha256"), sort_keys=True) for r in rows}) > 1:
            return done(UNVERIFIED, f"the {side} runs mix builds")
    if not ok_a:
        return done(NO_BASELINE, "the baseline has no successful run of this cell")
    if not ok_b:
        why = next((r.get("reason", "") for r in rows_b if r.get("status") != "ok"), "no successful run")
        return done(CANDIDATE_FAILED, why[:100])
    ia, ib = contract.identity(ok_a[0]), contract.identity(ok_b[0])
    for side, rows, ident in (("baseline", ok_a, ia), ("candidate", ok_b, ib)):
        if any(contract.identity(r) != ident for r in rows):
            return done(UNVERIFIED, f"the {side} runs differ in their workload identity")
    diff = [f for f in ia if ia[f] != ib[f]]
    if diff:
        return done(INCOMPARABLE, "the rows state different workloads: " + ", ".join(diff))
    fa, fb = len(rows_a) - len(ok_a), len(rows_b) - len(ok_b)
    da, db = [contract.derive_row(r) for r in ok_a], [contract.derive_row(r) for r in ok_b]
    for m in _metrics_for(ok_a[0], policy):
        xa = [d[m] for d in da if d[m] is not None]
        xb = [d[m] for d in db if d[m] is not None]
        cell["entries"].append(judge_metric(xa, xb, policy, m, fa, fb))
    v = worst(e["verdict"] for e in cell["entries"])
    first = next(e for e in cell["entries"] if e["verdict"] == v)
    return done(v, f"{first['metric']}" + (f": {first['note']}" if first["note"] else ""))


def compare_sets(rows_a: Iterable[dict], rows_b: Iterable[dict], policy: dict) -> List[dict]:
    ca, cb = _cells(rows_a), _cells(rows_b)
    keys = sorted(set(ca) | set(cb), key=lambda k: tuple("" if p is None else str(p) for p in k))
    return [compare_cell(k, ca.get(k), cb.get(k), policy) for k in keys]


def exit_code(cells: List[dict]) -> int:
    """1: a cell regressed, failed or is invalid.  2: nothing failed but something could not be verified, was not run
    or had no baseline (or nothing was compared).  0: every cell the baseline measured was compared, none worse."""
    vs = [c["verdict"] for c in cells if c["verdict"] != NEW]
    if any(v in FAILING for v in vs):
        return 1
    if not vs or any(v not in COMPARED for v in vs):
        return 2
    return 0


def render(cells: List[dict]) -> str:
    lines = ["| model | scenario | isl | osl | placement | storage | verdict | baseline (n) | candidate (n) | band | note |",
             "|---|---|---|---|---|---|---|---|---|---|---|"]
    for c in cells:
        h = c["entries"][0] if c["entries"] else {}
        num = lambda x: "-" if x is None else f"{x:.4g}"
        band = max((e["relative_band"] for e in c["entries"] if e.get("relative_band") is not None), default=None)
        lines.append("| " + " | ".join(str(p) for p in c["key"]) + f" | **{c['verdict']}** | {num(h.get('median_a'))} "
                     f"({h.get('n_a', 0)}) | {num(h.get('median_b'))} ({h.get('n_b', 0)}) | "
                     f"{'-' if band is None else f'{band:.1%}'} | {c['note']} |")
    return "\n".join(lines)
