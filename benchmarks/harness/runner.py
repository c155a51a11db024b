"""The runner for this package: one cell = one model, one scenario point, one repeat, through the public ``LLM`` API.

Every request is driven with exactly ``isl`` synthetic random in-vocabulary tokens (no chat template, prefix cache off:
random tokens defeat it and it would add order-dependent TTFT variance) and asked for exactly ``osl`` tokens with the
stop token ignored, single stream.  The runner records the raw window of each request - start, the host time each token
was delivered (the driver's step has synchronised by then: a token is delivered after its device-to-host copy), finish
and the executor steps it cost - and leaves every derived figure to ``contract.derive_row``.  A warm-up request of the
same shape runs first and is never measured.  Scenario definitions: the reference's benchmarks/README.md
("Scenario decode-curve", "Work-matched, tokenizer-neutral input", "Single-stream only").
"""
from __future__ import annotations

import hashlib
import json
import os
import random
import subprocess
import time
from pathlib import Path
from typing import Callable, Dict, List, Optional

from . import contract
from .observer import Observer

ROOT = Path(__file__).resolve().parents[2]


def _run(cmd: List[str]) -> str:
    try:
        return subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=20).stdout.strip()
    except Exception:
        return ""


def build_identity() -> Dict[str, object]:
    """Which build produced a row: commit (``-dirty`` with local changes), the digests of the loaded libraries, the
    compilers."""
    sha = _run(["git", "rev-parse", "HEAD"]) or "0" * 40
    if _run(["git", "status", "--porcelain", "--untracked-files=no"]):
        sha += "-dirty"
    libs = {}
    for so in sorted((ROOT / "poot_b200" / "lib").glob("*.so")):
        libs[so.name] = hashlib.sha256(so.read_bytes()).hexdigest()
    nv = _run(["nvcc", "--version"]).splitlines()
    import torch
    return {"build_sha": sha, "library_sha256": libs or {"none": "0" * 64},
            "nvcc_version": (nv[-2].strip() if len(nv) >= 2 else "unknown"), "torch_version": torch.__version__}


def checkpoint_digest(model: str, seed: int) -> str:
    if model.startswith("random:") or model == "fake":
        return f"random:seed={seed}"
    h = hashlib.sha256()
    p = Path(model)
    files = sorted(p.glob("*.safetensors")) + sorted(p.glob("*.gguf")) if p.is_dir() else [p]
    for f in files:                 # the whole weights set is read to the end: this also warms the page cache
        with open(f, "rb") as fh:
            while chunk := fh.read(1 << 24):
                h.update(chunk)
    return "sha256:" + h.hexdigest()


def open_model(model: str, rows: int, max_seq: int, seed: int, placement: str = "single"):
    """``fake`` (host engine), ``random:<preset>`` (random weights of a named architecture on the device) or a
    checkpoint path.  Single-device cells only: a multi-device cell is launched by the caller under
    ``torch.distributed.run`` with the server's placement flags."""
    from poot_b200.llm import LLM
    if placement != "single":
        raise ValueError("the in-process runner measures single-device cells")
    if model == "fake":
        return LLM.fake(rows=rows, max_seq=max_seq, num_blocks=max(256, rows * (max_seq // 16 + 2)), prefill_chunk=512)
    if model.startswith("random:"):
        return LLM.random(model.split(":", 1)[1], rows=rows, max_seq=max_seq, seed=seed)
    return LLM.load(model, rows=rows, max_seq=max_seq)


def measure_request(llm, prompt: List[int], osl: int, clock: Callable[[], float] = time.perf_counter) -> dict:
    from poot_b200.driver.sampler import SamplingParams
    times: List[float] = []
    steps0 = llm.driver.stats["steps"]
    params = SamplingParams(temperature=0.0, max_tokens=osl, ignore_eos=True)
    start = clock()
    llm.generate_tokens(prompt, params, on_token=lambda t: times.append(clock()))
    finish = clock()
    return {"prompt_tokens": len(prompt), "start": start, "token_times": times, "finish": finish,
            "steps": llm.driver.stats["steps"] - steps0}


def device_identity(llm) -> Dict[str, object]:
    import torch
    if llm.engine is not None and torch.cuda.is_available():
        name = torch.cuda.get_device_name(0)
        drv = _run(["nvidia-smi", "--query-gpu=driver_version", "--format=csv,noheader"]).splitlines()
        return {"device": name, "driver_version": drv[0] if drv else "unknown"}
    return {"device": "host", "driver_version": "none"}


def memory_classes(llm) -> Optional[Dict[str, int]]:
    """Bytes by class as the engine counts its own buffers (weights, K/V and recurrent state, workspace, staging)."""
    if llm.engine is None:
        return None
    from poot_b200.profile.memory import account
    inner = getattr(llm.driver.engine, "inner", llm.driver.engine)
    return account(llm.engine, inner).classes()


def run_cell(model: str, scenario: str, isl: int, osl: int, repeat: int = 1, requests: int = 1, rows: int = 1,
             seed: int = 0, storage_dtype: str = "bf16", observer: Optional[Observer] = None, llm=None) -> dict:
    """One row.  A failure to load or run is an ``error`` row with its reason, a workload the engine refuses a
    ``refused`` row; both still state the build."""
    row: Dict[str, object] = {"schema": contract.SCHEMA, "framework": "poot_b200", **build_identity(), "model": model,
                              "scenario": scenario, "isl": isl, "osl": osl, "repeat": repeat, "synthetic_tokens": True,
                              "prefix_cache": False, "placement": "single", "n_gpus": 1, "storage_dtype": storage_dtype,
                              "compute_dtype": "f32" if model == "fake" else "bf16"}
    obs = observer or Observer(device_probe=None)
    own = llm is None
    try:
        with obs:
            obs.mark("load")
            row["checkpoint_digest"] = checkpoint_digest(model, seed)
            if own:
                llm = open_model(model, rows, isl + osl + 16, seed)
            if own:
                llm.driver.prefix = None          # prefix cache off: no request may start from another's blocks
            row.update(device_identity(llm))
            vocab = llm.driver.vocab if hasattr(llm.driver, "vocab") else 1000
            rng = random.Random(seed * 7919 + repeat)
            prompt = lambda: [rng.randrange(3, vocab) for _ in range(isl)]
            obs.mark("warmup")
            measure_request(llm, prompt(), min(osl, 8))
            obs.mark("inference")
            row["requests"] = [measure_request(llm, prompt(), osl) for _ in range(requests)]
            mc = memory_classes(llm)
            if mc is not None:
                row["memory_classes"] = mc
        row["memory"] = obs.report()
        row["status"] = "ok"
        row.update({k: v for k, v in contract.derive_row(row).items()})
    except (ValueError, NotImplementedError) as e:
        row.update(status="refused", reason=f"{type(e).__name__}: {e}"[:300])
    except Exception as e:                                  # a crashed cell is a row, not a hole in the table
        row.update(status="error", reason=f"{type(e).__name__}: {e}"[:300])
    finally:
        if own and llm is not None:
            try:
                llm.close()
            except Exception:
                pass
    bad = contract.row_errors(row)
    if bad and row.get("status") == "ok":
        row.update(status="error", reason="the runner's own row is outside the contract: " + "; ".join(bad[:3]))
    return row


def append_row(run_dir: str, row: dict) -> None:
    os.makedirs(run_dir, exist_ok=True)
    with open(os.path.join(run_dir, "results.jsonl"), "a") as f:
        f.write(json.dumps(row) + "\n")


def load_rows(run_dir: str) -> List[dict]:
    p = Path(run_dir) / "results.jsonl"
    if not p.is_file():
        raise FileNotFoundError(f"{run_dir} holds no results.jsonl")
    return [json.loads(line) for line in p.read_text().splitlines() if line.strip()]
