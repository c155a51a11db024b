"""The result contract: what one benchmark row must state, and the ONE derivation of its timing figures.

A runner's JSON is untrusted input.  A row names the build, the device, the weights and the workload it measured, and
for every request the raw boundaries of its window (start, each delivered token, finish) plus the executor steps it
cost.  Everything a report shows - TTFT, the inter-token gaps, TPOT, finish, E2E, steady-state decode tokens/s - is
derived here from those boundaries and checked against any figure the runner also printed, so two runs compare on the
same arithmetic.  Definitions follow the reference's measurement contract (benchmarks/README.md "The measurement
contract": TPOT = (last token - first token) / (tokens - 1) with prefill and cleanup excluded; E2E = TTFT + sum(ITL) +
finish per request; a request that delivered N tokens cost at least N steps; summaries over fewer than 20 samples are
the median with the observed range) and its validator (benchmarks/harness/result_contract.py).
"""
from __future__ import annotations

import math
import re
import statistics
from typing import Dict, List, Optional, Sequence

SCHEMA = 1
SCENARIOS = ("decode-curve", "decode-128", "prefill-1k", "serve-load")
STATUSES = ("ok", "refused", "error")
BUILD_FIELDS = ("build_sha", "library_sha256", "nvcc_version", "torch_version")
MEASUREMENT_FIELDS = ("device", "driver_version", "n_gpus", "placement", "checkpoint_digest", "storage_dtype",
                      "compute_dtype")
WORKLOAD_FIELDS = ("model", "scenario", "isl", "osl", "synthetic_tokens", "prefix_cache")
MEMORY_CLASSES = ("weights_bytes", "kv_bytes", "workspace_bytes", "staging_bytes")
TAIL_SAMPLES = 20                       # below this many samples a percentile is the largest sample, not a tail
_TOL = 1e-9
_SHA = re.compile(r"[0-9a-f]{40}(-dirty)?")
_DIGEST = re.compile(r"(sha256:[0-9a-f]{64}|random:seed=\d+)")


def _finite(x) -> bool:
    return isinstance(x, (int, float)) and not isinstance(x, bool) and math.isfinite(x)


def _int(x) -> bool:
    return isinstance(x, int) and not isinstance(x, bool)


def request_errors(req: dict, requested: int) -> List[str]:
    """Why ``req`` is not an exact-work request window of ``requested`` tokens (empty list: it is one)."""
    errs: List[str] = []
    for f in ("start", "finish"):
        if not _finite(req.get(f)):
            errs.append(f"request.{f} must be a finite number; got {req.get(f)!r}")
    times = req.get("token_times")
    if not isinstance(times, list) or not all(_finite(t) for t in times):
        errs.append("request.token_times must be a list of finite numbers")
    if not _int(req.get("steps")) or req.get("steps", -1) < 0:
        errs.append(f"request.steps must be a nonnegative integer; got {req.get('steps')!r}")
    if errs:
        return errs
    n = len(times)
    if n != requested:
        errs.append(f"early stop: delivered {n} of {requested} requested tokens, so it cannot supply exact-work timing")
    seq = [req["start"], *times, req["finish"]]
    if any(b < a - _TOL for a, b in zip(seq, seq[1:])):
        errs.append("request boundaries are not in order (start <= tokens... <= finish)")
    if req["steps"] < n:
        errs.append(f"{n} tokens in {req['steps']} steps: a token was computed outside its request")
    return errs


def derive_request(req: dict) -> Dict[str, object]:
    """TTFT, the gaps, TPOT, finish and E2E of one validated request, in milliseconds, from its raw boundaries.
    Zero tokens: everything is finish.  One token: TTFT and finish, no gaps and no TPOT."""
    t0, t1, times = req["start"], req["finish"], req["token_times"]
    if not times:
        return {"ttft_ms": None, "itl_ms": [], "tpot_ms": None, "finish_ms": (t1 - t0) * 1e3, "e2e_ms": (t1 - t0) * 1e3}
    gaps = [(b - a) * 1e3 for a, b in zip(times, times[1:])]
    ttft = (times[0] - t0) * 1e3
    fin = (t1 - times[-1]) * 1e3
    return {"ttft_ms": ttft, "itl_ms": gaps, "tpot_ms": (sum(gaps) / len(gaps)) if gaps else None, "finish_ms": fin,
            "e2e_ms": ttft + sum(gaps) + fin}


def summarize(xs: Sequence[float]) -> Optional[Dict[str, float]]:
    """Median with the observed range; p90 / p99 only from ``TAIL_SAMPLES`` samples on."""
    xs = [x for x in xs if _finite(x)]
    if not xs:
        return None
    out = {"n": len(xs), "median": statistics.median(xs), "min": min(xs), "max": max(xs)}
    if len(xs) >= TAIL_SAMPLES:
        q = statistics.quantiles(xs, n=100, method="inclusive")
        out.update(p90=q[89], p99=q[98])
    return out


def derive_row(row: dict) -> Dict[str, object]:
    """The figures of an ``ok`` row from its requests: per-request medians, token-weighted gap summary, and the
    steady-state decode rate 1000 / median TPOT (never tokens / E2E, which folds prefill into the per-token rate)."""
    ds = [derive_request(r) for r in row["requests"]]
    tpots = [d["tpot_ms"] for d in ds if d["tpot_ms"] is not None]
    gaps = [g for d in ds for g in d["itl_ms"]]
    ttfts = [d["ttft_ms"] for d in ds if d["ttft_ms"] is not None]
    out: Dict[str, object] = {
        "ttft_ms": statistics.median(ttfts) if ttfts else None,
        "tpot_ms": statistics.median(tpots) if tpots else None,
        "itl_ms": summarize(gaps),
        "finish_ms": statistics.median([d["finish_ms"] for d in ds]) if ds else None,
        "e2e_ms": statistics.median([d["e2e_ms"] for d in ds]) if ds else None,
    }
    out["decode_tok_s"] = (1000.0 / out["tpot_ms"]) if out["tpot_ms"] else None
    out["prefill_tok_s"] = (row["isl"] / (out["ttft_ms"] / 1e3)) if out["ttft_ms"] else None
    return out


def memory_class_errors(mc) -> List[str]:
    if not isinstance(mc, dict) or not mc:
        return [f"memory_classes must be a nonempty object; got {mc!r}"]
    errs = [f"memory_classes names an unknown class {k!r}" for k in mc if k not in MEMORY_CLASSES]
    errs += [f"memory_classes.{k} must be a nonnegative integer; got {v!r}" for k, v in mc.items()
             if k in MEMORY_CLASSES and not (_int(v) and v >= 0)]
    return errs


def row_errors(row) -> List[str]:
    """Every reason ``row`` is not a result this harness will record or compare; an empty list accepts it."""
    if not isinstance(row, dict):
        return [f"a result row is a JSON object; got {type(row).__name__}"]
    errs: List[str] = []
    if row.get("schema") != SCHEMA:
        errs.append(f"schema must be {SCHEMA}; got {row.get('schema')!r}")
    if row.get("status") not in STATUSES:
        errs.append(f"status must be one of {STATUSES}; got {row.get('status')!r}")
    if row.get("scenario") not in SCENARIOS:
        errs.append(f"unknown scenario {row.get('scenario')!r}")
    for f in WORKLOAD_FIELDS:
        if f not in row:
            errs.append(f"workload field {f!r} is missing")
    for f in ("isl", "osl"):
        if f in row and not (_int(row[f]) and row[f] >= 0):
            errs.append(f"{f} must be a nonnegative integer; got {row[f]!r}")
    # a refusal states its build too: a row is attributable to one build whatever its status
    for f in BUILD_FIELDS:
        if not row.get(f):
            errs.append(f"build field {f!r} is missing")
    if row.get("build_sha") and not _SHA.fullmatch(str(row["build_sha"])):
        errs.append("build_sha must be a 40-digit git sha, optionally ending in '-dirty'")
    if row.get("status") != "ok":
        if not row.get("reason"):
            errs.append(f"a {row.get('status')} row states its reason")
        return errs
    for f in MEASUREMENT_FIELDS:
        if row.get(f) in (None, ""):
            errs.append(f"measurement field {f!r} is missing")
    if row.get("checkpoint_digest") and not _DIGEST.fullmatch(str(row["checkpoint_digest"])):
        errs.append("checkpoint_digest must be 'sha256:' and 64 hex digits, or 'random:seed=N' for random weights")
    reqs = row.get("requests")
    if not isinstance(reqs, list) or not reqs:
        errs.append("an ok row carries its requests' raw windows")
        return errs
    for i, r in enumerate(reqs):
        errs += [f"request {i}: {e}" for e in request_errors(r, row.get("osl", -1))]
    if errs:
        return errs
    d = derive_row(row)
    for f in ("ttft_ms", "tpot_ms", "e2e_ms", "decode_tok_s"):
        if f in row and row[f] is not None and d[f] is not None and not math.isclose(row[f], d[f], rel_tol=1e-6, abs_tol=1e-6):
            errs.append(f"{f} = {row[f]!r} disagrees with {d[f]!r} derived from the request windows")
    if "memory_classes" in row:
        errs += memory_class_errors(row["memory_classes"])
    mem = row.get("memory")
    if mem is not None:
        for f in ("peak_vram_bytes", "peak_rss_bytes"):
            if f in mem and mem[f] is not None and not (_int(mem[f]) and mem[f] >= 0):
                errs.append(f"memory.{f} must be a nonnegative integer; got {mem[f]!r}")
    return errs


def cell_key(row: dict):
    """The cell a row belongs to: what was measured on what, repeats excluded."""
    return (row.get("model"), row.get("scenario"), row.get("isl"), row.get("osl"), row.get("placement"),
            row.get("storage_dtype"))


def identity(row: dict) -> Dict[str, object]:
    """The fields two sets must agree on for their cell to be comparable at all."""
    return {f: row.get(f) for f in ("storage_dtype", "compute_dtype", "isl", "osl", "synthetic_tokens", "prefix_cache",
                                    "n_gpus", "placement", "device")}
