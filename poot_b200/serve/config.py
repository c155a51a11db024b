"""Serve configuration: typed, strictly parsed flags (an unknown option, an unparsable or out-of-bound value stops
start-up) - the flag set of the reference server (website/docs/serve/configuration.md:11-84;
crates/poot-serve/src/config.rs:87-484).  Execution choices are configuration, never environment variables.
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class ServeConfig:
    model: str = ""
    addr: str = "127.0.0.1:8080"
    placement: str = "single"            # single | tensor:0,1,.. | expert:0,1,.. | pipeline:0,1,..
    rows: int = 32
    max_seq: int = 4096
    prefill_chunk: int = 512
    prefill_budget: int = 0              # prefill tokens per step; 0 = one chunk (several chunks share a step when larger)
    kv_dtype: str = "bf16"
    matmul_precision: str = "narrow"
    chat_template: Optional[str] = None
    chat_template_file: Optional[str] = None
    draft_lookup: Optional[str] = None   # NGRAM:K
    draft_model: Optional[str] = None    # PATH:K - a smaller checkpoint proposes K tokens per verify step
    draft_mtp: int = 0                   # K tokens from the checkpoint's own multi-token-prediction heads (the checkpoint must store the layer)
    expert_pool: int = 0                 # > 0: resident experts per routed layer; the other experts stay in pinned host memory
    host_embedding: bool = False         # keep the token-embedding table in host memory; a step copies the rows it gathers
    check_ranges: bool = False           # prove every index of the step graphs in range before serving
    rate_limit_rpm: int = 0
    lora_admin_key_file: Optional[str] = None
    max_connections: int = 4096
    max_pending_requests: int = 256
    max_receiving_requests: int = 64
    max_queue_wait_secs: float = 60.0
    max_body_mib: int = 4
    max_image_body_mib: int = 64
    request_timeout_secs: float = 30.0
    write_timeout_secs: float = 30.0
    drain_timeout_secs: float = 30.0
    step_deadline_secs: float = 30.0     # a step still running after this is declared lost: the engine goes dead (0 = off)
    device_step_budget_secs: float = 5.0  # budget shared by all cross-rank waits inside one step's kernels
    ready_deadline_secs: float = 5.0     # multi-rank: every follower must say it is about to launch a step within this
    rank_heartbeat_timeout_secs: float = 3.0
    comm: str = "auto"                   # auto | fused | nccl: collectives of a tensor-parallel group
    device_timing: bool = False
    timing_max_steps: int = 4096
    timing_max_dispatch_records: int = 65536
    timing_max_in_flight_queries: int = 64
    timing_sample_every: int = 1
    prefix_cache: bool = True
    kv_fraction: float = 0.85            # share of free device memory given to the KV pool
    allowed_hosts: List[str] = field(default_factory=list)
    model_id: Optional[str] = None
    lora: Optional[str] = None           # PEFT adapter directory merged into the projections at load
    lora_slots: int = 0                  # > 0: resident adapters selected per request (POST /v1/lora_adapters, `model` = name)
    lora_max_rank: int = 64
    backend: str = "b200"                # b200 (the device engine) | graph (the general device executor; every family) | oracle (the CPU evaluator)

    def validate(self) -> None:
        def bound(name, lo, hi):
            v = getattr(self, name)
            if not (lo <= v <= hi):
                raise ValueError(f"--{name.replace('_', '-')} {v} outside [{lo}, {hi}]")
        bound("rows", 1, 1024); bound("max_seq", 128, 1 << 20); bound("prefill_chunk", 16, 8192)
        bound("max_pending_requests", 1, 1 << 16); bound("max_body_mib", 1, 1024); bound("kv_fraction", 0.05, 0.98)
        bound("max_queue_wait_secs", 0.1, 3600); bound("drain_timeout_secs", 0, 3600)
        bound("step_deadline_secs", 0, 3600); bound("device_step_budget_secs", 0, 600)
        bound("ready_deadline_secs", 0.05, 600); bound("rank_heartbeat_timeout_secs", 0.2, 600)
        if self.comm not in ("auto", "fused", "nccl"):
            raise ValueError(f"--comm {self.comm!r}: expected auto, fused or nccl")
        bound("timing_max_steps", 1, 1 << 24); bound("timing_max_dispatch_records", 1, 1 << 28)
        bound("timing_max_in_flight_queries", 1, 1 << 16); bound("timing_sample_every", 1, 1 << 20)
        bound("draft_mtp", 0, 16); bound("expert_pool", 0, 1 << 16)
        if sum(x is not None and x != 0 for x in (self.draft_lookup, self.draft_model, self.draft_mtp or None)) > 1:
            raise ValueError("one draft policy: --draft-lookup, --draft-model or --draft-mtp")
        if self.draft_model is not None:
            path, sep, k = self.draft_model.rpartition(":")
            if not sep or not path or not k.isdigit() or not (1 <= int(k) <= 16):
                raise ValueError(f"--draft-model {self.draft_model!r}: expected PATH:K with K in [1, 16]")
        if self.kv_dtype not in ("bf16", "f16", "f32"):
            raise ValueError(f"--kv-dtype {self.kv_dtype!r}: expected bf16, f16 or f32")
        if self.matmul_precision not in ("exact", "narrow", "split"):
            raise ValueError(f"--matmul-precision {self.matmul_precision!r}")
        if not (self.placement == "single" or self.placement.startswith(("tensor:", "expert:", "pipeline:"))):
            raise ValueError(f"--placement {self.placement!r}")
        host, _, port = self.addr.rpartition(":")
        if not host or not port.isdigit() or not (0 <= int(port) <= 65535):
            raise ValueError(f"address {self.addr!r} is not host:port")

    @property
    def placement_ordinals(self) -> List[int]:
        if self.placement == "single":
            return [0]
        return [int(x) for x in self.placement.split(":", 1)[1].split(",")]


class _StrictParser(argparse.ArgumentParser):
    def error(self, message):
        raise ValueError(message)


def parse_args(argv: List[str]) -> ServeConfig:
    p = _StrictParser(prog="poot-serve", allow_abbrev=False)
    p.add_argument("model")
    p.add_argument("addr", nargs="?", default="127.0.0.1:8080")
    d = ServeConfig()
    for name, val in vars(d).items():
        if name in ("model", "addr", "allowed_hosts"):
            continue
        flag = "--" + name.replace("_", "-")
        if isinstance(val, bool):
            p.add_argument(flag, action=argparse.BooleanOptionalAction, default=val)
        elif isinstance(val, int):
            p.add_argument(flag, type=int, default=val)
        elif isinstance(val, float):
            p.add_argument(flag, type=float, default=val)
        else:
            p.add_argument(flag, type=str, default=val)
    p.add_argument("--allowed-host", action="append", default=[])
    ns = p.parse_args(argv)
    kw = {k: v for k, v in vars(ns).items() if k != "allowed_host"}
    cfg = ServeConfig(**kw, allowed_hosts=ns.allowed_host)
    cfg.validate()
    return cfg
