"""Sampling parameters and their device encoding.

Defaults and knob semantics follow the reference CLI and host sampler (crates/poot-llm/src/bin/poot/generate.rs:
41-140; crates/poot-graph-ir/src/op.rs:118-189): temperature 0 = greedy; top-k 40, top-p 0.95, min-p 0.05 once a
temperature is set; the rule is chosen by ``rule_for_truncation``; the device reads
``params = (inv_temp, floor_offset, noise_scale, top_p)`` with ``floor_offset = ln(min_p) * temp`` (a logit is kept
when its probability is at least ``min_p`` of the top token's).  Logit adjustments are applied in the reference's
order: +bias, repetition (divide if > 0 else multiply), -presence, -frequency*count, +guided mask.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..oracle import sampling as S


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repeat_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None
    logit_bias: Dict[int, float] = field(default_factory=dict)
    max_tokens: int = 256
    stop_token_ids: List[int] = field(default_factory=list)
    stop: List[str] = field(default_factory=list)
    ignore_eos: bool = False
    logprobs: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def rule(self) -> int:
        if self.greedy:
            return S.GREEDY
        return S.rule_for_truncation(self.top_k, self.top_p)

    def device_params(self):
        """``(inv_temp, floor_offset, noise_scale, top_p)``."""
        if self.greedy:
            return (1.0, -math.inf, 0.0, 1.0)
        floor = math.log(self.min_p) * self.temperature if self.min_p > 0 else -1e30
        return (1.0 / self.temperature, max(floor, -1e30), 1.0, self.top_p)

    @property
    def needs_adjust(self) -> bool:
        return bool(self.logit_bias) or self.repeat_penalty != 1.0 or self.presence_penalty != 0.0 or \
            self.frequency_penalty != 0.0

    def validate(self) -> None:
        if self.temperature < 0 or not (0 <= self.top_p <= 1) or not (0 <= self.min_p <= 1) or self.top_k < 0:
            raise ValueError("sampling parameter out of range")
        if self.repeat_penalty <= 0:
            raise ValueError("repeat_penalty must be positive")
        if len(self.logit_bias) > 10000 or len(self.stop) > 16:
            raise ValueError("too many logit_bias entries or stop strings")


def step_seed(base_seed: int, step: int) -> int:
    """Per-token seed: the request seed advanced by the token index, hashed so rows never share noise."""
    return S.hash32(base_seed & 0xFFFFFFFF, step) & 0x7FFFFFFF
