"""Architecture description shared by the tracer, the CPU oracle and the device engine.

One ``DecoderConfig`` covers the "standard stack" families of the reference (embed -> layers of
``x += mixer(norm(x)); x += ffn(norm(x))`` -> final norm -> head; crates/poot-models/src/components/
standard.rs:618-866): llama / mistral / mixtral / qwen2 / qwen3 / qwen3moe / olmo2 / smollm3 / granite ...
Family modules fill it from an HF ``config.json`` or GGUF metadata.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Optional


@dataclass
class RopeScaling:
    """RoPE frequency scaling (crates/poot-graph-ir/src/rope_table.rs:64-150)."""
    kind: str = "none"  # none | linear | dynamic | yarn | longrope | llama3
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position: int = 8192
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    attention_factor: Optional[float] = None
    short_factor: Optional[list] = None
    long_factor: Optional[list] = None


@dataclass
class DecoderConfig:
    name: str = "llama"
    family: str = "llama"
    n_layers: int = 2
    hidden: int = 256
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 688
    vocab: int = 32000
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_dim: Optional[int] = None          # rotary channels (partial rotary); None = head_dim
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    max_position: int = 8192
    tie_embeddings: bool = False
    qk_norm: bool = False                   # per-head RMSNorm on q and k (qwen3)
    attn_bias: bool = False                 # q/k/v biases (qwen2)
    sliding_window: int = 0                 # 0 = full causal
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    # mixture of experts (0 experts = dense FFN)
    n_experts: int = 0
    top_k: int = 0
    moe_ffn: int = 0
    norm_topk_prob: bool = True             # softmax over the selected k only (mixtral) vs over all then pick
    embed_scale: float = 1.0
    residual_scale: float = 1.0
    logit_scale: float = 1.0
    bos_token: int = 1
    eos_token: int = 2

    @property
    def n_rep(self) -> int:
        return self.n_heads // self.n_kv_heads

    @property
    def q_size(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def rot(self) -> int:
        return self.head_dim if self.rope_dim is None else self.rope_dim

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    def param_count(self) -> int:
        per_layer = self.hidden * (self.q_size + 2 * self.kv_size) + self.q_size * self.hidden + 2 * self.hidden
        if self.is_moe:
            per_layer += self.n_experts * 3 * self.hidden * self.moe_ffn + self.hidden * self.n_experts
        else:
            per_layer += 3 * self.hidden * self.ffn
        head = 0 if self.tie_embeddings else self.vocab * self.hidden
        return self.n_layers * per_layer + self.vocab * self.hidden + head + self.hidden

    def to_dict(self) -> dict:
        return asdict(self)


def tiny_llama() -> DecoderConfig:
    """The tiny CPU-oracle configuration: 2 layers, hidden 256, 4/2 heads of 64, FFN 688, vocab 32000."""
    return DecoderConfig(name="tiny-llama", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=688,
                         vocab=32000, norm_eps=1e-5, rope_theta=10000.0, max_position=2048)


def llama3_8b() -> DecoderConfig:
    return DecoderConfig(name="llama-3-8b", n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                         ffn=14336, vocab=128256, norm_eps=1e-5, rope_theta=500000.0, max_position=8192,
                         bos_token=128000, eos_token=128001)


def llama3_70b() -> DecoderConfig:
    return DecoderConfig(name="llama-3-70b", n_layers=80, hidden=8192, n_heads=64, n_kv_heads=8, head_dim=128,
                         ffn=28672, vocab=128256, norm_eps=1e-5, rope_theta=500000.0, max_position=8192,
                         bos_token=128000, eos_token=128001)


def mixtral_8x7b() -> DecoderConfig:
    return DecoderConfig(name="mixtral-8x7b", family="mixtral", n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8,
                         head_dim=128, ffn=14336, vocab=32000, norm_eps=1e-5, rope_theta=1e6, max_position=32768,
                         n_experts=8, top_k=2, moe_ffn=14336)


PRESETS = {
    "tiny-llama": tiny_llama,
    "llama-3-8b": llama3_8b,
    "llama-3-70b": llama3_70b,
    "mixtral-8x7b": mixtral_8x7b,
}
