"""Checkpoint tensor names -> canonical weight roles, for HF safetensors and GGUF.

Canonical names are the ones the tracer declares (``layers.{i}.attn_q`` ...).  The tables follow the reference's
llama family (crates/poot-models/src/architectures/llama.rs:50-103): HF ``model.layers.N.self_attn.q_proj.weight``,
Mixtral ``block_sparse_moe.gate`` / ``experts.N.w1|w3|w2``; GGUF ``blk.N.attn_q.weight``, ``ffn_gate_inp``,
``ffn_{gate,up,down}_exps``.  GGUF llama files store Q and K rows permuted for interleaved RoPE; they are read back
into the half-split order (``GGUF_PAIRED_QK``, llama.rs:5-8).
"""
from __future__ import annotations

import re
from typing import Dict, Optional, Tuple

import numpy as np

HF_LAYER = {
    "input_layernorm.weight": "attn_norm", "self_attn.q_proj.weight": "attn_q", "self_attn.k_proj.weight": "attn_k",
    "self_attn.v_proj.weight": "attn_v", "self_attn.o_proj.weight": "attn_o", "self_attn.q_proj.bias": "attn_q_bias",
    "self_attn.k_proj.bias": "attn_k_bias", "self_attn.v_proj.bias": "attn_v_bias", "self_attn.q_norm.weight": "attn_q_norm",
    "self_attn.k_norm.weight": "attn_k_norm", "post_attention_layernorm.weight": "ffn_norm", "mlp.gate_proj.weight": "ffn_gate",
    "mlp.up_proj.weight": "ffn_up", "mlp.down_proj.weight": "ffn_down", "block_sparse_moe.gate.weight": "ffn_router",
    "mlp.gate.weight": "ffn_router",
}
HF_TOP = {"model.embed_tokens.weight": "embed", "model.norm.weight": "final_norm", "lm_head.weight": "lm_head"}
HF_EXPERT = {"w1": "gate", "w3": "up", "w2": "down", "gate_proj": "gate", "up_proj": "up", "down_proj": "down"}

GGUF_LAYER = {
    "attn_norm.weight": "attn_norm", "attn_q.weight": "attn_q", "attn_k.weight": "attn_k", "attn_v.weight": "attn_v",
    "attn_output.weight": "attn_o", "attn_q.bias": "attn_q_bias", "attn_k.bias": "attn_k_bias", "attn_v.bias": "attn_v_bias",
    "attn_q_norm.weight": "attn_q_norm", "attn_k_norm.weight": "attn_k_norm", "ffn_norm.weight": "ffn_norm",
    "ffn_gate.weight": "ffn_gate", "ffn_up.weight": "ffn_up", "ffn_down.weight": "ffn_down", "ffn_gate_inp.weight": "ffn_router",
}
GGUF_TOP = {"token_embd.weight": "embed", "output_norm.weight": "final_norm", "output.weight": "lm_head"}
GGUF_EXPERT = {"ffn_gate_exps.weight": "gate", "ffn_up_exps.weight": "up", "ffn_down_exps.weight": "down"}


def canonical_from_hf(name: str) -> Optional[str]:
    if name in HF_TOP:
        return HF_TOP[name]
    m = re.match(r"model\.layers\.(\d+)\.(.+)$", name)
    if not m:
        return None
    l, rest = m.group(1), m.group(2)
    if rest in HF_LAYER:
        return f"layers.{l}.{HF_LAYER[rest]}"
    e = re.match(r"(?:block_sparse_moe|mlp)\.experts\.(\d+)\.(\w+)\.weight$", rest)
    if e and e.group(2) in HF_EXPERT:
        return f"layers.{l}.experts.{e.group(1)}.{HF_EXPERT[e.group(2)]}"
    return None


def fused_hf_projection(name: str) -> Optional[Tuple[int, str]]:
    """``(layer, "qkv" | "gate_up")`` for the fused projection tensors some families store (Phi-3)."""
    m = re.match(r"model\.layers\.(\d+)\.(self_attn\.qkv_proj|mlp\.gate_up_proj)\.weight$", name)
    if not m:
        return None
    return int(m.group(1)), ("qkv" if m.group(2).endswith("qkv_proj") else "gate_up")


# rows a family's GGUF carries beside (or in place of) the shared ones (crates/poot-models/src/names/gguf.rs): OLMo 2
# stores the norms applied to each block's OUTPUT under the post-norm names; Gemma 2 / 3 have both pairs; gpt-oss names the
# norm before its feed-forward block ``post_attention_norm`` and has sinks, an output bias and a biased router
GGUF_FAMILY_LAYER = {
    "olmo2": {"post_attention_norm.weight": "attn_post_norm", "post_ffw_norm.weight": "ffn_post_norm"},
    "gemma2": {"post_attention_norm.weight": "attn_post_norm", "post_ffw_norm.weight": "ffn_post_norm"},
    "gemma3": {"post_attention_norm.weight": "attn_post_norm", "post_ffw_norm.weight": "ffn_post_norm"},
    "gpt_oss": {"post_attention_norm.weight": "ffn_norm", "attn_sinks.weight": "attn_sinks", "attn_output.bias": "attn_o_bias",
                "ffn_gate_inp.bias": "ffn_router_bias"},
    "bloom": {"attn_norm.bias": "attn_norm_bias", "ffn_norm.bias": "ffn_norm_bias", "attn_output.bias": "attn_o_bias",
              "ffn_up.bias": "ffn_up_bias", "ffn_down.bias": "ffn_down_bias"},
    "minimax_m2": {"exp_probs_b.bias": "ffn_router_select_bias"},
    "qwen38_27b": {"post_attention_norm.weight": "ffn_norm", "ssm_norm.weight": "gdn_gate_norm_w"},
    "gemma4": {"post_attention_norm.weight": "attn_post_norm", "post_ffw_norm.weight": "ffn_post_norm", "layer_output_scale.weight": "layer_scalar",
               "ffn_pre_norm_2.weight": "ffn_norm_2", "ffn_post_norm_1.weight": "ffn_post_norm_1", "ffn_post_norm_2.weight": "ffn_post_norm_2",
               "ffn_gate_inp.scale": "ffn_router_scale", "ffn_down_exps.scale": "ffn_expert_scale"},
    "deepseek2": {"attn_q_a.weight": "attn_q_a", "attn_q_a_norm.weight": "attn_q_a_norm", "attn_q_b.weight": "attn_q_b",
                  "attn_kv_a_mqa.weight": "attn_kv_a", "attn_kv_a_norm.weight": "attn_kv_a_norm", "attn_kv_b.weight": "attn_kv_b",
                  "ffn_gate_shexp.weight": "shared_gate", "ffn_up_shexp.weight": "shared_up", "ffn_down_shexp.weight": "shared_down",
                  "exp_probs_b.bias": "ffn_router_select_bias"},
}
# top-level rows of one family: BLOOM norms the embedding and its norms carry biases
GGUF_FAMILY_TOP = {
    "bloom": {"token_embd_norm.weight": "embed_norm", "token_embd_norm.bias": "embed_norm_bias", "output_norm.bias": "final_norm_bias"},
}
# fused rows a converter writes as one tensor: ``attn_qkv`` is q rows, then k rows, then v rows (llama.cpp regroups BLOOM's
# per-head interleaving into these thirds when it converts)
GGUF_FUSED_QKV = ("attn_qkv.weight", "attn_qkv.bias")
# families whose converter permutes Q / K rows for interleaved rotary pairs, read back half-split
GGUF_PAIRED_QK = ("llama", "mixtral", "smollm3")


def canonical_from_gguf(name: str, family: Optional[str] = None) -> Optional[str]:
    if name in GGUF_FAMILY_TOP.get(family or "", {}):
        return GGUF_FAMILY_TOP[family][name]
    if name in GGUF_TOP:
        return GGUF_TOP[name]
    m = re.match(r"blk\.(\d+)\.([^#]+)(?:#(\d+))?$", name)
    if not m:
        return None
    l, rest, ex = m.group(1), m.group(2), m.group(3)
    extra = GGUF_FAMILY_LAYER.get(family or "", {})
    if rest in extra:
        return f"layers.{l}.{extra[rest]}"
    if rest in GGUF_LAYER:
        return f"layers.{l}.{GGUF_LAYER[rest]}"
    if rest in GGUF_EXPERT and ex is not None:
        return f"layers.{l}.experts.{ex}.{GGUF_EXPERT[rest]}"
    return None


def gguf_qk_row_order(n_rows: int, n_heads: int) -> np.ndarray:
    """Row gather that turns a GGUF (interleaved-pair) Q/K matrix back into half-split order."""
    hd = n_rows // n_heads
    idx = np.arange(n_rows).reshape(n_heads, hd // 2, 2)
    return idx.transpose(0, 2, 1).reshape(-1)


def hf_to_gguf_qk_row_order(n_rows: int, n_heads: int) -> np.ndarray:
    """The permutation llama.cpp's converter applies to HF Q/K rows (inverse of ``gguf_qk_row_order``)."""
    hd = n_rows // n_heads
    idx = np.arange(n_rows).reshape(n_heads, 2, hd // 2)
    return idx.transpose(0, 2, 1).reshape(-1)


def gdn_grouped_heads(n_value_heads: int, n_key_heads: int) -> np.ndarray:
    """llama.cpp stores a gated delta net's value heads tiled over the key heads: position ``t`` holds the head that the
    source checkpoint, which groups value heads by key head, has at ``(t % key_heads) * rep + t // key_heads``
    (crates/poot-models/src/components/gdn_names.rs:283-297).  Returns that index per tiled position."""
    rep = n_value_heads // n_key_heads
    t = np.arange(n_value_heads)
    return (t % n_key_heads) * rep + t // n_key_heads
