"""Device and pinned-host memory counted by what a buffer is for.

Roles follow the reference's ``BufferRole`` (crates/poot-runtime-common/src/memory.rs:11-31): ``weight``, ``state``
(K/V pools, recurrent and convolution state, the sparse indexer's key pool), ``activation`` (a step's intermediate
values and scratch), ``input`` / ``output`` (what a step binds and what is read back), ``meta`` (tables, counters,
control blocks) and ``staging`` (pinned host buffers and bounce buffers that bridge transfers).  ``account`` walks an
engine once after construction; tensors that share storage are counted once.  The totals feed ``/metrics`` and the
benchmark rows' ``memory_classes``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, Set

import torch

ROLES = ("weight", "state", "activation", "input", "output", "meta", "staging")
_STATE = ("gdn_state", "gdn_conv_state", "ssm_state", "ssm_conv_state", "idx_pool")
_INPUT = ("tokens", "positions", "slots", "row_seq", "row_ctx", "logit_idx", "block_tables", "samp_params", "samp_topk",
          "samp_seeds", "adj_idx", "adj_val", "guided_mask", "embed_rows", "embed_flags", "rope_cos_tok", "rope_sin_tok",
          "carry_in", "seg_table", "mtp_first")
_OUTPUT = ("picked", "logprobs", "logits", "carry_out")
_META = ("cos", "sin", "cos_local", "sin_local", "cos_none", "sin_none", "argmax_scratch", "mtp_zero")


@dataclass
class MemoryCounters:
    bytes_by_role: Dict[str, int] = field(default_factory=lambda: {r: 0 for r in ROLES})
    _seen: Set[int] = field(default_factory=set)

    def add(self, role: str, tensors: Iterable) -> None:
        if role not in self.bytes_by_role:
            raise ValueError(f"unknown buffer role {role!r}")
        for t in tensors:
            for x in _leaves(t):
                key = x.untyped_storage().data_ptr() if x.numel() else 0
                if key == 0 or key in self._seen:
                    continue
                self._seen.add(key)
                self.bytes_by_role[role] += x.untyped_storage().nbytes()

    @property
    def total(self) -> int:
        return sum(self.bytes_by_role.values())

    def classes(self) -> Dict[str, int]:
        """The four classes a benchmark row states."""
        b = self.bytes_by_role
        return {"weights_bytes": b["weight"], "kv_bytes": b["state"],
                "workspace_bytes": b["activation"] + b["input"] + b["output"] + b["meta"], "staging_bytes": b["staging"]}


def _leaves(t):
    if t is None:
        return
    if isinstance(t, torch.Tensor):
        yield t
    elif hasattr(t, "tensors") and callable(t.tensors):             # PlanarWeight
        yield from t.tensors()
    elif hasattr(t, "packed") and isinstance(t.packed, torch.Tensor):   # QuantWeight
        yield t.packed
    elif isinstance(t, dict):
        for v in t.values():
            yield from _leaves(v)
    elif isinstance(t, (list, tuple)):
        for v in t:
            yield from _leaves(v)


def account(engine, step_engine=None) -> MemoryCounters:
    """Counters of a ``DecoderEngine`` (and the pinned buffers of the step engine in front of it)."""
    m = MemoryCounters()
    w = engine.w
    m.add("weight", [w.embed, w.final_norm, w.lm_head, w.final_norm_b, w.embed_norm, w.embed_norm_b, w.mtp])
    for L in w.layers:
        m.add("weight", [v for v in vars(L).values()])
    m.add("state", [engine.kv.buf] + [getattr(engine, n, None) for n in _STATE])
    m.add("input", [getattr(engine, n, None) for n in _INPUT])
    m.add("output", [getattr(engine, n, None) for n in _OUTPUT])
    m.add("meta", [getattr(engine, n, None) for n in _META])
    prog = getattr(engine, "program", None)
    if prog is not None:
        m.add("activation", [prog.arena])
    hosted = getattr(engine, "_hosted", None)
    if hosted:
        m.add("staging", [hosted.get("stage"), hosted.get("table")])
        m.add("input", [hosted.get("slot")])
    m.add("activation", [v for k, v in vars(engine).items() if isinstance(v, (torch.Tensor, dict, list, tuple)) and
                         not k.startswith("_graphs")])
    if step_engine is not None:
        m.add("staging", [v for k, v in vars(step_engine).items() if k.startswith("h_") and isinstance(v, torch.Tensor)])
    return m
