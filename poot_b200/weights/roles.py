"""``WeightRole`` names what a tensor is for; ``WeightId`` = (role, layer, expert); ``WeightMap`` resolves ids to the
stored tensors of a checkpoint through the canonical names of the family tables; ``rank_view`` cuts a tensor-parallel
share following the Megatron layouts (q/k/v/gate/up split on ``out``, o/down split on ``in``, norms, embeddings and
the router replicated; the head split on the vocabulary)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, Iterable, Optional, Tuple


class WeightRole(Enum):
    EMBED = "embed"
    LM_HEAD = "lm_head"
    FINAL_NORM = "final_norm"
    ATTN_NORM = "attn_norm"
    ATTN_Q = "attn_q"
    ATTN_K = "attn_k"
    ATTN_V = "attn_v"
    ATTN_O = "attn_o"
    ATTN_Q_BIAS = "attn_q_bias"
    ATTN_K_BIAS = "attn_k_bias"
    ATTN_V_BIAS = "attn_v_bias"
    ATTN_Q_NORM = "attn_q_norm"
    ATTN_K_NORM = "attn_k_norm"
    FFN_NORM = "ffn_norm"
    FFN_GATE = "ffn_gate"
    FFN_UP = "ffn_up"
    FFN_DOWN = "ffn_down"
    MOE_ROUTER = "ffn_router"
    MOE_GATE = "gate"
    MOE_UP = "up"
    MOE_DOWN = "down"
    LORA_A = "lora_a"
    LORA_B = "lora_b"


SPLIT_OUT = {WeightRole.ATTN_Q, WeightRole.ATTN_K, WeightRole.ATTN_V, WeightRole.FFN_GATE, WeightRole.FFN_UP,
             WeightRole.ATTN_Q_BIAS, WeightRole.ATTN_K_BIAS, WeightRole.ATTN_V_BIAS, WeightRole.LM_HEAD}
SPLIT_IN = {WeightRole.ATTN_O, WeightRole.FFN_DOWN}
UNSUPPORTED_ROLE_FAMILIES = ("mla", "mamba2", "gdn", "kda", "dsa", "mtp")   # roles of families that are refused by the registry


@dataclass(frozen=True)
class WeightId:
    role: WeightRole
    layer: Optional[int] = None
    expert: Optional[int] = None

    @property
    def canonical(self) -> str:
        if self.layer is None:
            return self.role.value
        if self.expert is not None:
            return f"layers.{self.layer}.experts.{self.expert}.{self.role.value}"
        return f"layers.{self.layer}.{self.role.value}"

    @staticmethod
    def parse(name: str) -> "WeightId":
        parts = name.split(".")
        if parts[0] != "layers":
            return WeightId(WeightRole(name))
        layer = int(parts[1])
        if parts[2] == "experts":
            return WeightId(WeightRole(parts[4]), layer, int(parts[3]))
        return WeightId(WeightRole(".".join(parts[2:])), layer)


class WeightMap:
    """id -> stored tensor view (zero-copy views of the mapped checkpoint)."""

    def __init__(self, canonical: Dict[str, object]):
        self._by_id: Dict[WeightId, object] = {}
        self.unknown = []
        for name, w in canonical.items():
            try:
                self._by_id[WeightId.parse(name)] = w
            except (ValueError, IndexError):
                self.unknown.append(name)

    def __getitem__(self, wid: WeightId):
        return self._by_id[wid]

    def __contains__(self, wid: WeightId) -> bool:
        return wid in self._by_id

    def __len__(self) -> int:
        return len(self._by_id)

    def ids(self) -> Iterable[WeightId]:
        return self._by_id.keys()

    def missing(self, cfg) -> list:
        """Ids a decoder of ``cfg`` needs that the checkpoint does not have."""
        need = [WeightId(WeightRole.EMBED), WeightId(WeightRole.FINAL_NORM)]
        for l in range(cfg.n_layers):
            for r in (WeightRole.ATTN_NORM, WeightRole.ATTN_Q, WeightRole.ATTN_K, WeightRole.ATTN_V, WeightRole.ATTN_O,
                      WeightRole.FFN_NORM):
                need.append(WeightId(r, l))
            if cfg.is_moe:
                need.append(WeightId(WeightRole.MOE_ROUTER, l))
                for e in range(cfg.n_experts):
                    need += [WeightId(r, l, e) for r in (WeightRole.MOE_GATE, WeightRole.MOE_UP, WeightRole.MOE_DOWN)]
            else:
                need += [WeightId(r, l) for r in (WeightRole.FFN_GATE, WeightRole.FFN_UP, WeightRole.FFN_DOWN)]
        return [w for w in need if w not in self]


def rank_view(role: WeightRole, shape: Tuple[int, ...], rank: int, world: int) -> Tuple[slice, ...]:
    """Index expression of rank ``rank``'s share of a ``shape``-d tensor of ``role``."""
    if world == 1 or (role not in SPLIT_OUT and role not in SPLIT_IN):
        return tuple(slice(None) for _ in shape)
    axis = 0 if role in SPLIT_OUT else 1
    if shape[axis] % world:
        raise ValueError(f"{role.value} extent {shape[axis]} does not divide over {world} ranks")
    n = shape[axis] // world
    return tuple(slice(rank * n, (rank + 1) * n) if a == axis else slice(None) for a in range(len(shape)))
