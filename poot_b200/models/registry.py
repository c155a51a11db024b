"""Family registry: HF ``model_type`` / GGUF ``general.architecture`` -> configuration builder and name tables.

Counterpart of the reference registry (crates/poot-models/src/registry.rs:383-426): the family is resolved
from the checkpoint header before any weight is read.  Families whose layer is the standard stack share one
tracer (``Model``); what differs is how a ``DecoderConfig`` is read from the header and how checkpoint tensor
names map to canonical weight roles.  Families outside the standard stack (MLA, state-space mixers, encoders,
vision towers) are listed with a typed refusal so a load names what is missing instead of failing obscurely.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

from .config import DecoderConfig, RopeScaling
from .model import Model


class UnsupportedFamily(ValueError):
    """The checkpoint names a family this build has no tracer for (typed refusal, named capability)."""


@dataclass
class FamilyEntry:
    name: str
    hf_types: List[str]
    gguf_archs: List[str]
    from_hf: Optional[Callable[[dict], DecoderConfig]]
    missing: Optional[str] = None     # capability that is not built when the family is refused


def _rope_scaling(c: dict) -> RopeScaling:
    rs = c.get("rope_scaling") or {}
    kind = rs.get("rope_type", rs.get("type", "none")) or "none"
    if kind == "default":
        kind = "none"
    return RopeScaling(kind=kind, factor=float(rs.get("factor", 1.0)),
                       low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                       high_freq_factor=float(rs.get("high_freq_factor", 4.0)),
                       original_max_position=int(rs.get("original_max_position_embeddings",
                                                        c.get("original_max_position_embeddings", 8192))),
                       beta_fast=float(rs.get("beta_fast", 32.0)), beta_slow=float(rs.get("beta_slow", 1.0)),
                       attention_factor=rs.get("attention_factor"), short_factor=rs.get("short_factor"),
                       long_factor=rs.get("long_factor"))


def _base(c: dict, family: str, **over) -> DecoderConfig:
    H, nh = c["hidden_size"], c["num_attention_heads"]
    cfg = DecoderConfig(
        name=c.get("_name_or_path", family) or family, family=family, n_layers=c["num_hidden_layers"], hidden=H,
        n_heads=nh, n_kv_heads=c.get("num_key_value_heads", nh), head_dim=c.get("head_dim") or H // nh,
        ffn=c.get("intermediate_size", 4 * H), vocab=c["vocab_size"], norm_eps=float(c.get("rms_norm_eps", 1e-6)),
        rope_theta=float(c.get("rope_theta", 10000.0)), rope_scaling=_rope_scaling(c),
        max_position=int(c.get("max_position_embeddings", 8192)), tie_embeddings=bool(c.get("tie_word_embeddings", False)),
        sliding_window=int(c.get("sliding_window") or 0) if c.get("use_sliding_window", True) else 0,
        bos_token=c.get("bos_token_id", 1) or 1, eos_token=(c.get("eos_token_id", 2) if isinstance(c.get("eos_token_id", 2), int) else c["eos_token_id"][0]))
    for k, v in over.items():
        setattr(cfg, k, v)
    return cfg


def _llama(c: dict) -> DecoderConfig:
    if c.get("attention_bias") or c.get("mlp_bias"):
        raise UnsupportedFamily("llama with attention_bias / mlp_bias")   # as the reference (llama.rs:152-156)
    cfg = _base(c, "llama")
    if c.get("num_local_experts", 0) > 0:   # Mixtral rides the llama entry (llama.rs:136-208)
        cfg.family, cfg.n_experts, cfg.top_k, cfg.moe_ffn = "mixtral", c["num_local_experts"], c["num_experts_per_tok"], c["intermediate_size"]
    return cfg


def _qwen2(c): return _base(c, "qwen2", attn_bias=True, sliding_window=0)
def _qwen3(c): return _base(c, "qwen3", qk_norm=True, sliding_window=0)
def _smollm3(c): return _base(c, "smollm3")
def _olmo2(c): return _base(c, "olmo2", qk_norm=True)
def _phi3(c): return _base(c, "phi3")


def _qwen3moe(c):
    return _base(c, "qwen3moe", qk_norm=True, sliding_window=0, n_experts=c["num_experts"], top_k=c["num_experts_per_tok"],
                 moe_ffn=c["moe_intermediate_size"], norm_topk_prob=bool(c.get("norm_topk_prob", True)))


def _granite(c):
    return _base(c, "granite", embed_scale=float(c.get("embedding_multiplier", 1.0)),
                 residual_scale=float(c.get("residual_multiplier", 1.0)),
                 logit_scale=1.0 / float(c.get("logits_scaling", 1.0)))


def _olmoe(c):
    return _base(c, "olmoe", qk_norm=True, n_experts=c["num_experts"], top_k=c["num_experts_per_tok"],
                 moe_ffn=c["intermediate_size"], norm_topk_prob=bool(c.get("norm_topk_prob", False)))


SHIPPED: List[FamilyEntry] = [
    FamilyEntry("qwen2", ["qwen2"], ["qwen2"], _qwen2),
    FamilyEntry("llama", ["llama", "mistral", "mixtral"], ["llama"], _llama),
    FamilyEntry("qwen3", ["qwen3"], ["qwen3"], _qwen3),
    FamilyEntry("olmo2", ["olmo2"], ["olmo2"], _olmo2),
    FamilyEntry("phi3", ["phi3"], ["phi3"], _phi3),
    FamilyEntry("smollm3", ["smollm3"], ["smollm3"], _smollm3),
    FamilyEntry("granite", ["granite", "granitemoe"], ["granite"], _granite),
    FamilyEntry("qwen3moe", ["qwen3_moe"], ["qwen3moe"], _qwen3moe),
    FamilyEntry("olmoe", ["olmoe"], ["olmoe"], _olmoe),
    # families the reference ships whose mixers are not built here: refused by name
    FamilyEntry("mpt", ["mpt"], ["mpt"], None, "ALiBi attention + LayerNorm stack"),
    FamilyEntry("bloom", ["bloom"], ["bloom"], None, "ALiBi attention + LayerNorm stack"),
    FamilyEntry("gemma2", ["gemma2"], ["gemma2"], None, "sandwich norms, GeGLU, logit softcap"),
    FamilyEntry("gemma3", ["gemma3", "gemma3_text"], ["gemma3"], None, "sandwich norms, GeGLU, dual rope bases"),
    FamilyEntry("gemma4", ["gemma4"], ["gemma4"], None, "per-layer embeddings, proportional rope"),
    FamilyEntry("gpt_oss", ["gpt_oss"], ["gpt-oss"], None, "attention sinks, MXFP4 experts, clamped SwiGLU"),
    FamilyEntry("minimax_m2", ["minimax_m2"], ["minimax-m2"], None, "sigmoid router with bias"),
    FamilyEntry("deepseek2", ["deepseek_v2"], ["deepseek2"], None, "multi-head latent attention"),
    FamilyEntry("deepseek3", ["deepseek_v3"], ["deepseek2"], None, "multi-head latent attention, group-limited routing"),
    FamilyEntry("deepseek32", ["deepseek_v32"], ["deepseek32"], None, "sparse attention indexer"),
    FamilyEntry("deepseek4", ["deepseek_v4"], ["deepseek4"], None, "compressed attention"),
    FamilyEntry("nemotron_h", ["nemotron_h"], ["nemotron_h"], None, "Mamba2 mixer"),
    FamilyEntry("bert", ["bert"], ["bert"], None, "bidirectional encoder"),
    FamilyEntry("idefics3", ["idefics3"], [], None, "vision tower"),
    FamilyEntry("qwen3next", ["qwen3_next"], ["qwen3next"], None, "gated delta-net mixer"),
    FamilyEntry("qwen38", ["qwen3_8"], ["qwen38"], None, "gated delta-net mixer"),
    FamilyEntry("qwen38_27b", ["qwen3_8_27b"], ["qwen38"], None, "gated delta-net mixer"),
    FamilyEntry("glm53_flash", ["glm5_flash"], ["glm53"], None, "kimi delta attention"),
    FamilyEntry("qwen_vl", ["qwen2_5_vl"], ["qwen2vl"], None, "vision tower, sectioned mRoPE"),
]


class Registry:
    def __init__(self, entries: Optional[List[FamilyEntry]] = None):
        self.entries = list(entries if entries is not None else SHIPPED)

    @staticmethod
    def builtin() -> "Registry":
        return Registry()

    def resolve_hf(self, config: dict) -> Model:
        mt = config.get("model_type")
        for e in self.entries:
            if mt in e.hf_types:
                if e.from_hf is None:
                    raise UnsupportedFamily(f"family {e.name!r} needs {e.missing}, which this build does not have")
                return Model(e.from_hf(config))
        raise UnsupportedFamily(f"no family for model_type {mt!r}")

    def resolve_gguf(self, arch: str, meta: dict) -> Model:
        from ..load.gguf import config_from_gguf_metadata
        for e in self.entries:
            if arch in e.gguf_archs:
                if e.from_hf is None:
                    raise UnsupportedFamily(f"family {e.name!r} needs {e.missing}, which this build does not have")
                return Model(config_from_gguf_metadata(arch, meta, e.name))
        raise UnsupportedFamily(f"no family for GGUF architecture {arch!r}")

    def supported(self) -> List[str]:
        return [e.name for e in self.entries if e.from_hf is not None]

    def listed(self) -> List[str]:
        return [e.name for e in self.entries]
