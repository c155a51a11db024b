"""Placement of one model over the GPUs of a node (crates/poot-llm/src/driver/placement.rs:28).

``single`` | ``tensor:0,1,..`` (Megatron tensor parallelism, one process per listed ordinal) | ``expert:0,1,..``
(experts split over the ranks, attention tensor-parallel over the same ranks) | ``pipeline:0,1,..`` (contiguous layer
ranges, one stage per listed ordinal, cut so that the heaviest stage is as light as possible with the embedding on
the first stage and the head on the last; placement.rs:1-16,126-160).
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
        return {"single": [], "tensor": [Feature.TENSOR_PLACEMENT], "expert": [Feature.EXPERT_PLACEMENT],
                "pipeline": [Feature.PIPELINE_PLACEMENT]}[self.kind]

    @staticmethod
    def parse(text: str) -> "Placement":
        if text == "single":
            return Placement("single")
        kind, sep, rest = text.partition(":")
        if kind not in ("tensor", "expert", "pipeline") or not sep:
            raise PlacementError(f"placement {text!r}: expected single, tensor:<ordinals>, expert:<ordinals> or pipeline:<ordinals>")
        try:
            ords = tuple(int(x) for x in rest.split(","))
        except ValueError:
            raise PlacementError(f"placement {text!r}: ordinals must be integers") from None
        if len(set(ords)) != len(ords) or any(o < 0 for o in ords):
            raise PlacementError(f"placement {text!r}: ordinals must be distinct and non-negative")
        if kind != "pipeline" and len(ords) & (len(ords) - 1):
            raise PlacementError(f"placement {text!r}: the group size must be a power of two")
        return Placement(kind, ords)

    def validate(self, cfg: DecoderConfig) -> None:
        """Divisibility rules of the Megatron layouts (crates/poot-graph-plan/src/passes/sharding.rs:219-251)."""
        w = self.world
        if w == 1:
            return
        if self.kind == "pipeline":
            if cfg.n_layers < w:
                raise PlacementError(f"{cfg.n_layers} layers cannot fill {w} pipeline stages")
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


def layer_bytes(cfg: DecoderConfig, layer: int, bytes_per_weight: float = 2.0) -> int:
    """Resident weight bytes of one layer (what the cut balance weighs)."""
    H = cfg.hidden
    n = H * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * H + 2 * H
    if cfg.moe_layer(layer):
        n += cfg.n_experts * 3 * H * cfg.moe_ffn + H * cfg.n_experts + 3 * H * cfg.shared_width
    else:
        n += (3 if cfg.gated_ffn else 2) * H * cfg.ffn
    return int(n * bytes_per_weight)


def pipeline_cuts(cfg: DecoderConfig, stages: int, bytes_per_weight: float = 2.0) -> list:
    """Contiguous layer ranges ``[(l0, l1)] * stages`` minimising the heaviest stage, every stage non-empty, with the
    token embedding counted on the first stage and the head (when it is not tied) on the last.  Exact dynamic
    programme over the prefix sums (the reference balances the same way, placement.rs:126-160,227)."""
    L = cfg.n_layers
    if not (1 <= stages <= L):
        raise PlacementError(f"{L} layers cannot fill {stages} pipeline stages")
    w = [layer_bytes(cfg, l, bytes_per_weight) for l in range(L)]
    pre = [0]
    for x in w:
        pre.append(pre[-1] + x)
    emb = int(cfg.vocab * cfg.hidden * bytes_per_weight)
    head = 0 if cfg.tie_embeddings else emb

    def cost(s: int, a: int, b: int) -> int:
        c = pre[b] - pre[a]
        if s == 0:
            c += emb
        if s == stages - 1:
            c += head if not cfg.tie_embeddings else (emb if stages > 1 else 0)
        return c

    INF = float("inf")
    best = [[INF] * (L + 1) for _ in range(stages + 1)]
    arg = [[0] * (L + 1) for _ in range(stages + 1)]
    best[0][0] = 0
    for s in range(1, stages + 1):
        for b in range(s, L - (stages - s) + 1):
            for a in range(s - 1, b):
                if best[s - 1][a] == INF:
                    continue
                c = max(best[s - 1][a], cost(s - 1, a, b))
                if c < best[s][b]:
                    best[s][b], arg[s][b] = c, a
    cuts, b = [], L
    for s in range(stages, 0, -1):
        a = arg[s][b]
        cuts.append((a, b))
        b = a
    return cuts[::-1]
