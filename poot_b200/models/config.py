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
    kind: str = "none"  # none | linear | dynamic | yarn | longrope | llama3 | proportional
    factor: float = 1.0
    proportion: float = 1.0          # proportional: share of the head's channel pairs that rotate (the rest keep frequency 0)
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
    norm_topk_prob: bool = True             # gates of the selected experts are renormalised to sum to one (mixtral); False: softmax over all, as is
    embed_scale: float = 1.0
    residual_scale: float = 1.0
    logit_scale: float = 1.0
    # --- what differs between the standard-stack families (components/standard.rs:618-650, attention.rs, ffn.rs) ---
    norm_kind: str = "rms"                  # rms | layer
    norm_bias: bool = False                 # LayerNorm carries a bias (bloom)
    block: str = "pre"                      # pre: x += f(norm(x)) | post: x += norm(f(x)) (olmo2) | sandwich: x += norm(f(norm(x)))
    qk_norm_wide: bool = False              # with qk_norm: one RMSNorm over the whole q / k projection (olmo2, olmoe)
    act: str = "silu"                       # silu | gelu_tanh | gelu_erf
    gated_ffn: bool = True                  # False: down(act(up(x))) (mpt, bloom)
    out_bias: bool = False                  # bias on the attention output projection
    mlp_bias: bool = False                  # biases on the FFN projections
    pos: str = "rope"                       # rope | alibi | none
    alibi_slopes: str = "bloom"             # bloom (closest power of two + extras) | mpt
    alibi_bias_max: float = 8.0
    attn_scale: Optional[float] = None      # None = 1/sqrt(head_dim)
    layer_windows: Optional[list] = None    # per-layer sliding window (0 = full); None = sliding_window everywhere
    rope_theta_local: Optional[float] = None  # rope base of the windowed layers when it differs (gemma3)
    embed_norm: bool = False                # LayerNorm right after the embedding (bloom)
    attn_sinks: bool = False                # one learned logit per head joins every softmax (gpt-oss)
    swiglu_limit: float = 0.0               # >0: clamped SwiGLU (gpt-oss): gate<=limit, |up|<=limit, (up+1)*gate*sigmoid(alpha*gate)
    swiglu_alpha: float = 1.702
    router: str = "softmax"                 # softmax | sigmoid
    router_bias: bool = False               # linear bias on the router logits (gpt-oss)
    router_select_bias: bool = False        # per-expert bias added for selection only (minimax-m2, deepseek3)
    n_group: int = 1                        # group-limited routing (deepseek3): experts in n_group groups, keep topk_group groups
    topk_group: int = 1
    routed_scale: float = 1.0
    n_shared_experts: int = 0               # always-on experts of width n_shared_experts * moe_ffn (deepseek)
    first_dense_layers: int = 0             # leading layers with a dense FFN in a MoE model (deepseek)
    expert_bias: bool = False               # biases on the expert projections (gpt-oss)
    # multi-head latent attention (deepseek2/3): 0 = off
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    qk_nope_dim: int = 0
    qk_rope_dim: int = 0
    v_head_dim: int = 0
    # hybrid stacks (nemotron-h, qwen3-next): per-layer token mixer and whether an FFN follows it
    layer_kinds: Optional[list] = None      # "attention" | "mamba" | "gdn" | "none" per layer; None = attention everywhere
    layer_ffn: Optional[list] = None        # 1 = the layer has an FFN after its mixer; None = every layer has one
    dense_layers: Optional[list] = None     # layers of a MoE model whose FFN is dense (besides the leading first_dense_layers)
    # multi-token prediction: layers the checkpoint stores after the text stack, each guessing one token further ahead
    # from a position's closing hidden state and the token that follows it (DeepSeek-V3 ``num_nextn_predict_layers``)
    mtp_layers: int = 0
    mtp_head: bool = False                  # this configuration IS such a layer (``mtp_config``): its input mixes a carry in
    ssm_heads: int = 0                      # Mamba2: heads, head width, state size, B/C groups, conv taps
    ssm_head_dim: int = 0
    ssm_state: int = 0
    ssm_groups: int = 1
    ssm_conv: int = 4
    ssm_conv_bias: bool = True
    gdn_k_heads: int = 0                    # gated delta net: key heads, value heads, head width, conv taps
    gdn_v_heads: int = 0
    gdn_head_dim: int = 0
    gdn_conv: int = 4
    attn_gate: bool = False                 # attention output multiplied by sigmoid of a per-channel gate projection (qwen3-next)
    shared_expert_gate: bool = False        # shared expert scaled by sigmoid(x . w) (qwen3-next)
    shared_ffn: int = 0                     # width of the shared expert when it is not n_shared_experts * moe_ffn
    norm_offset: float = 0.0                # checkpoint stores norm weights as w - offset (gemma: 1.0); added at load
    rope_layers: Optional[list] = None      # per-layer flag: 1 = rotary applied, 0 = no position signal (smollm3 NoPE layers)
    rope_interleaved: bool = False          # checkpoint stores rotary channels as interleaved pairs (deepseek): rows are re-ordered at load
    latent_norm_eps: Optional[float] = None  # epsilon of the norms inside latent attention (None: norm_eps)
    index_topk: int = 0                     # sparse attention: keys each query keeps, picked by the indexer (0: dense attention)
    index_n_heads: int = 0
    index_head_dim: int = 0
    # gated hyper-connections (Qwen3.8-Flash-Next): the residual is ``hc_count`` parallel streams; every block reads a
    # gated mean of their grouped norm and writes back into each stream with its own weight (0: one plain stream)
    hc_count: int = 0
    hc_lowrank: int = 0
    index_ratio: int = 0                    # block indexer: positions per scored block (0: the per-position indexer)
    index_budget: int = 0                   # block indexer: positions kept per query (``index_budget // index_ratio`` blocks)
    gdn_gate_act: str = "silu"              # activation of the delta-net output gate: silu | sigmoid
    # per-layer hashed n-gram embedding blocks in front of some layers, in ordinal order (``models/ngram.py``)
    ple_layers: Optional[list] = None
    ple_embed_dim: int = 0
    ple_conv: int = 0
    ngram_size: int = 0
    heads_per_ngram: int = 0
    ngram_vocab_base: int = 0
    ngram_divisible_by: int = 1
    ngram_seed: int = 1234
    mrope_sections: Optional[list] = None   # channel pairs of the time / row / column rotary streams (Qwen2.5-VL); None: one stream
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

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    def window_of(self, layer: int) -> int:
        return self.sliding_window if self.layer_windows is None else int(self.layer_windows[layer])

    def mixer_of(self, layer: int) -> str:
        return "attention" if self.layer_kinds is None else self.layer_kinds[layer]

    def has_ffn(self, layer: int) -> bool:
        return self.layer_ffn is None or bool(self.layer_ffn[layer])

    @property
    def is_recurrent(self) -> bool:
        return self.layer_kinds is not None and any(k in ("mamba", "gdn") for k in self.layer_kinds)

    @property
    def shared_width(self) -> int:
        return self.shared_ffn or self.n_shared_experts * self.moe_ffn

    def ple_tables(self, layer: int):
        """Hash constants of the n-gram block in front of ``layer`` (``None``: the layer has none)."""
        if not self.ple_layers or layer not in self.ple_layers:
            return None
        from .ngram import ngram_tables
        return ngram_tables(self.ple_layers.index(layer), self.ngram_size, self.heads_per_ngram, self.ngram_vocab_base,
                            self.ngram_divisible_by, self.ngram_seed, self.vocab)

    def uses_rope(self, layer: int) -> bool:
        return self.pos == "rope" and (self.rope_layers is None or bool(self.rope_layers[layer]))

    def moe_layer(self, layer: int) -> bool:
        return self.is_moe and layer >= self.first_dense_layers and not (self.dense_layers and layer in self.dense_layers)

    @property
    def plain_block(self) -> bool:
        """The pre-norm SwiGLU rope layer the fused tensor-parallel programs are written for."""
        return (self.block == "pre" and self.act == "silu" and not self.qk_norm_wide and self.rope_theta_local is None
                and (self.rope_layers is None or all(self.rope_layers)) and self.final_softcap == 0
                and self.layer_kinds is None and not self.attn_gate and not self.is_mla and not self.attn_sinks
                and not self.out_bias and not self.expert_bias and self.swiglu_limit == 0 and not self.router_bias
                and self.norm_kind == "rms" and self.gated_ffn and self.pos == "rope" and not self.embed_norm)

    @property
    def mla_eps(self) -> float:
        return self.norm_eps if self.latent_norm_eps is None else self.latent_norm_eps

    def device_gaps(self) -> list:
        """Features of this configuration that the device program does not implement (empty = runs on the device);
        the CPU oracle evaluates all of them."""
        g = []
        if self.index_topk and (self.index_n_heads > 64 or self.index_head_dim > 256 or self.index_head_dim < self.qk_rope_dim):
            g.append("sparse attention indexer beyond 64 heads of width 256")
        if self.norm_kind != "rms" and self.block != "pre": g.append("LayerNorm with a post norm")
        if self.block != "pre" and self.is_moe: g.append(f"{self.block}-norm block with routed experts")
        if self.gated_ffn and self.act not in ("silu", "gelu_tanh", "gelu_erf"): g.append(f"{self.act} gated FFN")
        if self.is_moe and self.act not in ("silu", "relu2", "gelu_tanh", "gelu_erf"): g.append(f"{self.act} experts")
        if self.mlp_bias and self.gated_ffn: g.append("biases of a gated dense FFN")
        if self.out_bias and self.block != "pre": g.append("output bias with a post norm")
        if self.swiglu_limit > 0 and not self.is_moe: g.append("clamped SwiGLU in a dense FFN")
        if self.router == "softmax" and self.router_select_bias: g.append("router variant")
        if self.n_group > 32 or (self.n_group > 1 and self.router != "sigmoid"): g.append("group-limited routing outside the sigmoid router")
        if self.shared_width and self.gated_ffn and self.act != "silu": g.append("gated shared expert that is not SwiGLU")
        if self.is_moe and self.top_k > 16: g.append("more than 16 experts per token")
        if self.is_mla and (self.qk_rope_dim % 2 or (self.qk_nope_dim + self.qk_rope_dim) % 32 or self.v_head_dim % 32):
            g.append("latent attention head widths that are not multiples of 32")
        if self.ssm_heads and self.ssm_head_dim not in (32, 64, 128): g.append(f"Mamba2 head width {self.ssm_head_dim}")
        if self.ssm_heads and self.ssm_conv not in (2, 3, 4): g.append(f"conv width {self.ssm_conv}")
        if self.gdn_k_heads and self.gdn_head_dim not in (64, 128): g.append(f"delta-net head width {self.gdn_head_dim}")
        if self.hc_count: g.append("gated hyper-connection residual streams")
        if self.index_ratio: g.append("block-indexed sparse attention")
        if self.ple_layers: g.append("hashed n-gram embedding blocks")
        if self.head_dim % 32 or not (32 <= self.head_dim <= 512): g.append(f"head_dim {self.head_dim}")
        return g

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


def mtp_config(cfg: DecoderConfig) -> DecoderConfig:
    """The configuration of ``cfg``'s multi-token-prediction layer as a one-layer model of its own: the block has the
    kind the layer after the text stack would have (attention mixer; routed FFN when the stack's last layers are), its
    closing norm is the layer's ``shared_head.norm`` and its embedding and head are the target's."""
    from dataclasses import replace
    if cfg.mtp_layers < 1:
        raise ValueError(f"{cfg.family} stores no multi-token-prediction layer")
    n = cfg.n_layers
    moe = cfg.is_moe and n >= cfg.first_dense_layers
    win = cfg.layer_windows[-1] if getattr(cfg, "layer_windows", None) else None
    return replace(cfg, name=cfg.name + "-mtp", n_layers=1, first_dense_layers=0 if moe else 1, dense_layers=None,
                   layer_kinds=None, layer_ffn=None, layer_windows=[win] if win is not None else None, mtp_layers=0,
                   mtp_head=True)


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
