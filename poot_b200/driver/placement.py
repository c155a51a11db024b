"""Placement of one model over the GPUs of a node (crates/poot-llm/src/driver/placement.rs:28).

``single`` | ``tensor:0,1,..`` (Megatron tensor parallelism, one process per listed ordinal) | ``expert:0,1,..``
(experts split over the ranks, attention tensor-parallel over the same ranks) | ``pipeline:..`` (typed refusal).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

from ..models.config import DecoderConfig
from .features import Feature, Unavailable, UNAVAILABLE


class PlacementError(ValueError):
    pass


@dataclass(frozen=True)
class Placement:
    kind: str                 # "single" | "tensor" | "expert"
    ordinals: tuple = (0,)

    @property
    def world(self) -> int:
        return len(self.ordinals)

    @property
    def features(self) -> List[Feature]:
        return {"single": [], "tensor": [Feature.TENSOR_PLACEMENT], "expert": [Feature.EXPERT_PLACEMENT]}[self.kind]

    @staticmethod
    def parse(text: str) -> "Placement":
        if text == "single":
            return Placement("single")
        kind, sep, rest = text.partition(":")
        if kind == "pipeline":
            raise Unavailable(Feature.PIPELINE_PLACEMENT, UNAVAILABLE[Feature.PIPELINE_PLACEMENT])
        if kind not in ("tensor", "expert") or not sep:
            raise PlacementError(f"placement {text!r}: expected single, tensor:<ordinals> or expert:<ordinals>")
        try:
            ords = tuple(int(x) for x in rest.split(","))
        except ValueError:
            raise PlacementError(f"placement {text!r}: ordinals must be integers") from None
        if len(set(ords)) != len(ords) or any(o < 0 for o in ords):
            raise PlacementError(f"placement {text!r}: ordinals must be distinct and non-negative")
        if len(ords) & (len(ords) - 1):
            raise PlacementError(f"placement {text!r}: the group size must be a power of two")
        return Placement(kind, ords)

    def validate(self, cfg: DecoderConfig) -> None:
        """Divisibility rules of the Megatron layouts (crates/poot-graph-plan/src/passes/sharding.rs:219-251)."""
        w = self.world
        if w == 1:
            return
        if cfg.n_heads % w:
            raise PlacementError(f"{cfg.n_heads} query heads do not divide over {w} ranks")
        if cfg.n_kv_heads % w and w % cfg.n_kv_heads:
            raise PlacementError(f"{cfg.n_kv_heads} KV heads neither divide over nor replicate onto {w} ranks")
        if cfg.vocab % w:
            raise PlacementError(f"vocabulary {cfg.vocab} does not divide over {w} ranks")
        if self.kind == "tensor" and not cfg.is_moe and (cfg.ffn % w or (cfg.ffn // w) % 64):
            raise PlacementError(f"FFN width {cfg.ffn} does not split into 64-aligned shares over {w} ranks")
        if self.kind == "expert":
            if not cfg.is_moe:
                raise PlacementError("expert placement needs a mixture-of-experts family")
            if cfg.n_experts % w:
                raise PlacementError(f"{cfg.n_experts} experts do not divide over {w} ranks")
