"""Feature composition: ONE compatibility table decides which serving features may be combined.

Every pairing the engine cannot run is a row here with its reason, so a refused configuration fails at startup
with a typed error instead of somewhere inside a step (crates/poot-llm/src/driver/features.rs:1-13).
"""
from __future__ import annotations

from enum import Enum
from typing import Iterable, List, Tuple


class Feature(Enum):
    TENSOR_PLACEMENT = "tensor placement"
    EXPERT_PLACEMENT = "expert placement"
    PIPELINE_PLACEMENT = "pipeline placement"
    DRAFT_LOOKUP = "lookup drafting"
    DRAFT_MODEL = "draft model"
    DRAFT_MTP = "multi-token-prediction drafting"
    BEAM = "beam search"
    GUIDED = "guided decoding"
    LOGPROBS = "logprobs"
    ADAPTERS = "LoRA adapters"
    PACKED_WEIGHTS = "packed (block-quantised) weights"
    DEVICE_TIMING = "per-kernel device timing"
    PREFIX_CACHE = "prefix cache"
    RECURRENT_STATE = "recurrent state"
    EXPERT_POOL = "pooled experts"


class Incompatible(ValueError):
    def __init__(self, a: Feature, b: Feature, why: str):
        super().__init__(f"{a.value} cannot be combined with {b.value}: {why}")
        self.pair, self.why = (a, b), why


class Unavailable(ValueError):
    def __init__(self, f: Feature, why: str):
        super().__init__(f"{f.value} is not available: {why}")
        self.feature, self.why = f, why


F = Feature
TABLE: List[Tuple[Feature, Feature, str]] = [
    (F.TENSOR_PLACEMENT, F.EXPERT_PLACEMENT, "one placement per model; expert placement already shards attention over the same ranks"),
    (F.TENSOR_PLACEMENT, F.BEAM, "beam search reads whole-vocabulary logits on the host; tensor ranks hold vocabulary shards"),
    (F.EXPERT_PLACEMENT, F.BEAM, "beam search reads whole-vocabulary logits on the host; ranks hold vocabulary shards"),
    (F.TENSOR_PLACEMENT, F.DEVICE_TIMING, "event brackets between launches would serialise ranks that wait on one another in-kernel"),
    (F.EXPERT_PLACEMENT, F.DEVICE_TIMING, "event brackets between launches would serialise ranks that wait on one another in-kernel"),
    (F.TENSOR_PLACEMENT, F.DRAFT_MODEL, "the draft model would need its own rank group"),
    (F.DRAFT_LOOKUP, F.DRAFT_MODEL, "one draft policy per driver"),
    (F.DRAFT_MTP, F.DRAFT_LOOKUP, "one draft policy per driver"),
    (F.DRAFT_MTP, F.DRAFT_MODEL, "one draft policy per driver"),
    (F.DRAFT_MTP, F.BEAM, "speculation verifies one greedy continuation"),
    (F.DRAFT_MTP, F.GUIDED, "a constraint mask is computed one token ahead, not for k drafted positions"),
    (F.DRAFT_MTP, F.PREFIX_CACHE, "the layer's cache entry of a block's last position depends on the token after it"),
    (F.DRAFT_MTP, F.ADAPTERS, "the layer reads the base model's hidden state"),
    (F.DRAFT_MTP, F.TENSOR_PLACEMENT, "the layer runs on the single-device engine"),
    (F.DRAFT_MTP, F.EXPERT_PLACEMENT, "the layer runs on the single-device engine"),
    (F.DRAFT_MTP, F.PIPELINE_PLACEMENT, "the layer runs on the single-device engine"),
    (F.DRAFT_LOOKUP, F.BEAM, "speculation verifies one greedy continuation"),
    (F.DRAFT_MODEL, F.BEAM, "speculation verifies one greedy continuation"),
    (F.DRAFT_LOOKUP, F.GUIDED, "a constraint mask is computed one token ahead, not for k drafted positions"),
    (F.DRAFT_MODEL, F.GUIDED, "a constraint mask is computed one token ahead, not for k drafted positions"),
    (F.BEAM, F.GUIDED, "beams would each need a clone of the constraint state"),
    (F.PACKED_WEIGHTS, F.EXPERT_PLACEMENT, "packed expert weights have no fused grouped kernel"),
    (F.RECURRENT_STATE, F.PREFIX_CACHE, "a prefix hit skips tokens; the recurrent state after them is not in the K/V cache"),
    (F.RECURRENT_STATE, F.BEAM, "a fork would need a copy of the recurrent state; only K/V blocks are copied"),
    (F.RECURRENT_STATE, F.TENSOR_PLACEMENT, "recurrent mixers run on the host evaluator, in one process"),
    (F.ADAPTERS, F.TENSOR_PLACEMENT, "the adapter bank is built for the single-device engine"),
    (F.ADAPTERS, F.EXPERT_PLACEMENT, "the adapter bank is built for the single-device engine"),
    (F.ADAPTERS, F.PIPELINE_PLACEMENT, "the adapter bank is built for the single-device engine"),
    (F.PIPELINE_PLACEMENT, F.TENSOR_PLACEMENT, "one placement per model: stages are not themselves tensor-parallel groups"),
    (F.PIPELINE_PLACEMENT, F.EXPERT_PLACEMENT, "one placement per model: stages are not themselves expert-parallel groups"),
    (F.PIPELINE_PLACEMENT, F.DEVICE_TIMING, "per-launch device spans are recorded on one device"),
    (F.PIPELINE_PLACEMENT, F.BEAM, "a fork copies K/V blocks on every stage; only the leader's copy is wired"),
    (F.ADAPTERS, F.PACKED_WEIGHTS, "adapter deltas are applied to bf16 projections"),
    (F.EXPERT_POOL, F.TENSOR_PLACEMENT, "the expert pool is built for the single-device engine"),
    (F.EXPERT_POOL, F.EXPERT_PLACEMENT, "an expert-parallel group keeps its experts resident on their ranks"),
    (F.EXPERT_POOL, F.PIPELINE_PLACEMENT, "the expert pool is built for the single-device engine"),
    (F.EXPERT_POOL, F.PACKED_WEIGHTS, "packed expert weights have no fused grouped kernel"),
]
UNAVAILABLE: dict = {}      # features no build of the engine offers (none at present); a model that lacks what a feature
#                             needs is refused where the model is known (``require_mtp``)


def require_mtp(cfg) -> None:
    """Typed refusal of multi-token-prediction drafting on a model whose checkpoint stores no such layer."""
    if getattr(cfg, "mtp_layers", 0) < 1:
        raise Unavailable(F.DRAFT_MTP, f"{getattr(cfg, 'family', 'this model')} stores no multi-token-prediction layer")


def check(features: Iterable[Feature]) -> None:
    """Raises ``Unavailable`` / ``Incompatible`` for the first offending feature or pair."""
    fs = list(dict.fromkeys(features))
    for f in fs:
        if f in UNAVAILABLE:
            raise Unavailable(f, UNAVAILABLE[f])
    have = set(fs)
    for a, b, why in TABLE:
        if a in have and b in have:
            raise Incompatible(a, b, why)
