"""Hugging Face checkpoint tensors -> canonical weight roles, per family.

The tracer declares canonical names (``layers.{i}.attn_q``, ``layers.{i}.experts.{e}.gate`` ...); this module maps
what a family's checkpoint stores onto them (the reference keeps one name table per architecture module,
crates/poot-models/src/architectures/*.rs).  Most tensors map one to one and stay zero-copy views of the mmapped
file.  The exceptions are rewritten once at load:

* fused projections are cut into row views (Phi-3 ``qkv_proj`` / ``gate_up_proj``, MPT ``Wqkv``, the stacked
  ``experts.gate_up_proj[E, 2F, H]`` tensors newer checkpoints use);
* Bloom's ``query_key_value`` is stored per head as ``(q, k, v)`` triples and is de-interleaved;
* gpt-oss experts are stored ``[E, H, 2F]`` with gate and up columns alternating; they are transposed into
  checkpoint order (``[out, in]``) with the gate rows first;
* Gemma norm weights are stored as ``w - 1`` and get the one added;
* DeepSeek stores rotary channels as interleaved pairs; the rows that produce them are re-ordered into the
  half-split order the rotary op uses (a common permutation of q and k channels leaves q.k unchanged).
"""
from __future__ import annotations

import re
from dataclasses import replace
from typing import Callable, Dict, Optional

import numpy as np

from ..models.config import DecoderConfig
from ..quant.formats import descriptor
from ..quant.weights import PackedWeight, WeightStore


class CheckpointLayout(ValueError):
    """A tensor the family's table expects is missing or has the wrong extent."""


def f32_weight(name: str, a: np.ndarray) -> PackedWeight:
    a = np.ascontiguousarray(a, dtype=np.float32)
    return PackedWeight(name, "F32", tuple(a.shape), a.view(np.uint8).reshape(-1))


def first_axis(w: PackedWeight, i: int) -> PackedWeight:
    """``w[i]`` of a stacked tensor as a view (dense and block formats are contiguous per leading index)."""
    d = descriptor(w.format)
    if d.storage == "planar":
        raise CheckpointLayout(f"{w.name}: stacked planar tensors are not cut")
    inner = int(np.prod(w.shape[1:]))
    nbytes = inner // d.block_elems * d.block_bytes
    raw = w.payload.reshape(-1)
    return PackedWeight(f"{w.name}[{i}]", w.format, tuple(w.shape[1:]), raw[i * nbytes:(i + 1) * nbytes])


# llama-like layer tensors; families override single entries
LAYER = {
    "input_layernorm.weight": "attn_norm", "post_attention_layernorm.weight": "ffn_norm",
    "self_attn.q_proj.weight": "attn_q", "self_attn.k_proj.weight": "attn_k", "self_attn.v_proj.weight": "attn_v",
    "self_attn.o_proj.weight": "attn_o", "self_attn.q_proj.bias": "attn_q_bias", "self_attn.k_proj.bias": "attn_k_bias",
    "self_attn.v_proj.bias": "attn_v_bias", "self_attn.o_proj.bias": "attn_o_bias",
    "self_attn.q_norm.weight": "attn_q_norm", "self_attn.k_norm.weight": "attn_k_norm", "self_attn.sinks": "attn_sinks",
    "mlp.gate_proj.weight": "ffn_gate", "mlp.up_proj.weight": "ffn_up", "mlp.down_proj.weight": "ffn_down",
    "mlp.gate_proj.bias": "ffn_gate_bias", "mlp.up_proj.bias": "ffn_up_bias", "mlp.down_proj.bias": "ffn_down_bias",
    "block_sparse_moe.gate.weight": "ffn_router", "mlp.gate.weight": "ffn_router", "mlp.router.weight": "ffn_router",
    "mlp.router.bias": "ffn_router_bias", "block_sparse_moe.router.layer.weight": "ffn_router",
    "mlp.gate.e_score_correction_bias": "ffn_router_select_bias", "mlp.e_score_correction_bias": "ffn_router_select_bias",
    "block_sparse_moe.e_score_correction_bias": "ffn_router_select_bias",
    "mlp.shared_experts.gate_proj.weight": "shared_gate", "mlp.shared_experts.up_proj.weight": "shared_up",
    "mlp.shared_experts.down_proj.weight": "shared_down",
    "mlp.shared_expert.gate_proj.weight": "shared_gate", "mlp.shared_expert.up_proj.weight": "shared_up",
    "mlp.shared_expert.down_proj.weight": "shared_down", "mlp.shared_expert_gate.weight": "shared_expert_gate",
    # multi-head latent attention
    "self_attn.q_a_proj.weight": "attn_q_a", "self_attn.q_a_layernorm.weight": "attn_q_a_norm",
    "self_attn.q_b_proj.weight": "attn_q_b", "self_attn.kv_a_proj_with_mqa.weight": "attn_kv_a",
    "self_attn.kv_a_layernorm.weight": "attn_kv_a_norm", "self_attn.kv_b_proj.weight": "attn_kv_b",
    # sparse attention indexer
    "self_attn.indexer.wq_b.weight": "idx_q", "self_attn.indexer.wk.weight": "idx_k", "self_attn.indexer.k_norm.weight": "idx_k_norm",
    "self_attn.indexer.k_norm.bias": "idx_k_norm_bias", "self_attn.indexer.weights_proj.weight": "idx_weights",
}
# norm placement differs by block kind: the same checkpoint name means a different role
POST_BLOCK = {"post_attention_layernorm.weight": "attn_post_norm", "post_feedforward_layernorm.weight": "ffn_post_norm"}
SANDWICH_BLOCK = {"input_layernorm.weight": "attn_norm", "post_attention_layernorm.weight": "attn_post_norm",
                  "pre_feedforward_layernorm.weight": "ffn_norm", "post_feedforward_layernorm.weight": "ffn_post_norm"}
TOP = {"model.embed_tokens.weight": "embed", "model.norm.weight": "final_norm", "lm_head.weight": "lm_head",
       "model.language_model.embed_tokens.weight": "embed", "model.language_model.norm.weight": "final_norm"}
# tensors a checkpoint stores for its multi-token-prediction layer beside that layer's block (DeepSeek-V3 layout:
# ``model.layers.<n_layers>.*``); the block's own tensors map like any layer's
MTP = {"enorm.weight": "mtp.enorm", "hnorm.weight": "mtp.hnorm", "eh_proj.weight": "mtp.eh_proj",
       "shared_head.norm.weight": "mtp.head_norm", "shared_head.head.weight": "mtp.lm_head",
       "embed_tokens.weight": "mtp.embed"}
EXPERT = {"w1": "gate", "w3": "up", "w2": "down", "gate_proj": "gate", "up_proj": "up", "down_proj": "down"}

MPT_LAYER = {"norm_1.weight": "attn_norm", "norm_2.weight": "ffn_norm", "attn.out_proj.weight": "attn_o",
             "ffn.up_proj.weight": "ffn_up", "ffn.down_proj.weight": "ffn_down"}
BLOOM_LAYER = {"input_layernorm.weight": "attn_norm", "input_layernorm.bias": "attn_norm_bias",
               "post_attention_layernorm.weight": "ffn_norm", "post_attention_layernorm.bias": "ffn_norm_bias",
               "self_attention.dense.weight": "attn_o", "self_attention.dense.bias": "attn_o_bias",
               "mlp.dense_h_to_4h.weight": "ffn_up", "mlp.dense_h_to_4h.bias": "ffn_up_bias",
               "mlp.dense_4h_to_h.weight": "ffn_down", "mlp.dense_4h_to_h.bias": "ffn_down_bias"}
BLOOM_TOP = {"transformer.word_embeddings.weight": "embed", "transformer.word_embeddings_layernorm.weight": "embed_norm",
             "transformer.word_embeddings_layernorm.bias": "embed_norm_bias", "transformer.ln_f.weight": "final_norm",
             "transformer.ln_f.bias": "final_norm_bias", "lm_head.weight": "lm_head"}


def _deinterleave_rows(n: int) -> np.ndarray:
    """Row order that turns ``(x0, y0, x1, y1, ...)`` pairs into the half-split ``(x0, x1, ..., y0, y1, ...)``."""
    return np.concatenate([np.arange(0, n, 2), np.arange(1, n, 2)])


BERT_TOP = {"embeddings.word_embeddings.weight": "embed", "embeddings.position_embeddings.weight": "embed_pos",
            "embeddings.token_type_embeddings.weight": "embed_type", "embeddings.LayerNorm.weight": "embed_norm",
            "embeddings.LayerNorm.bias": "embed_norm_bias", "pooler.dense.weight": "pooler", "pooler.dense.bias": "pooler_bias",
            "classifier.weight": "classifier", "classifier.bias": "classifier_bias"}
BERT_LAYER = {"attention.self.query": "attn_q", "attention.self.key": "attn_k", "attention.self.value": "attn_v",
              "attention.output.dense": "attn_o", "attention.output.LayerNorm": "attn_post_norm",
              "intermediate.dense": "ffn_up", "output.dense": "ffn_down", "output.LayerNorm": "ffn_post_norm"}


def _map_bert(cfg, store: WeightStore) -> Dict[str, PackedWeight]:
    canon: Dict[str, PackedWeight] = {}
    for n in store.names():
        short = n[5:] if n.startswith("bert.") else n
        if short in BERT_TOP:
            canon[BERT_TOP[short]] = store[n]
            continue
        m = re.match(r"encoder\.layer\.(\d+)\.(.+)\.(weight|bias)$", short)
        if m and m.group(2) in BERT_LAYER:
            canon[f"layers.{m.group(1)}.{BERT_LAYER[m.group(2)]}" + ("_bias" if m.group(3) == "bias" else "")] = store[n]
    return canon


VISION_TOP = {"embeddings.patch_embedding.bias": "patch_embed_bias", "embeddings.position_embedding.weight": "pos_embed",
              "post_layernorm.weight": "post_norm", "post_layernorm.bias": "post_norm_bias"}
VISION_LAYER = {"layer_norm1": "attn_norm", "layer_norm2": "ffn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
                "self_attn.v_proj": "attn_v", "self_attn.out_proj": "attn_o", "mlp.fc1": "ffn_up", "mlp.fc2": "ffn_down"}


class _Renamed:
    """A weight store seen through a name prefix swap (a text stack nested one level down in a multimodal checkpoint)."""

    def __init__(self, store: WeightStore, old: str, new: str):
        self.store = store
        self.inner = {(new + n[len(old):] if n.startswith(old) else n): n for n in store.names()}

    def names(self):
        return list(self.inner)

    def __getitem__(self, name: str) -> PackedWeight:
        return self.store[self.inner[name]]


def _map_vision(store: WeightStore) -> Dict[str, PackedWeight]:
    """Vision tower and connector tensors of an Idefics3 / SmolVLM checkpoint (``model.vision_model.*``,
    ``model.connector.*``); the patch convolution ``[out, C, p, p]`` flattens to a matrix over flattened patches."""
    canon: Dict[str, PackedWeight] = {}
    for n in store.names():
        if n == "model.connector.modality_projection.proj.weight":
            canon["vision.projector"] = store[n]
            continue
        if not n.startswith("model.vision_model."):
            continue
        short = n[len("model.vision_model."):]
        if short == "embeddings.patch_embedding.weight":
            w = store[n].to_f32()
            canon["vision.patch_embed"] = f32_weight("vision.patch_embed", w.reshape(w.shape[0], -1))
        elif short in VISION_TOP:
            canon["vision." + VISION_TOP[short]] = store[n]
        else:
            m = re.match(r"encoder\.layers\.(\d+)\.(.+)\.(weight|bias)$", short)
            if m and m.group(2) in VISION_LAYER:
                canon[f"vision.layers.{m.group(1)}.{VISION_LAYER[m.group(2)]}" + ("_bias" if m.group(3) == "bias" else "")] = store[n]
    return canon


GEMMA4_TOP = {"embed_tokens.weight": "embed", "norm.weight": "final_norm", "embed_tokens_per_layer.weight": "ple_embed",
              "per_layer_model_projection.weight": "ple_model_proj", "per_layer_projection_norm.weight": "ple_proj_norm"}
GEMMA4_LAYER = {"input_layernorm.weight": "attn_norm", "post_attention_layernorm.weight": "attn_post_norm",
                "pre_feedforward_layernorm.weight": "ffn_norm", "post_feedforward_layernorm.weight": "ffn_post_norm",
                "self_attn.q_proj.weight": "attn_q", "self_attn.k_proj.weight": "attn_k", "self_attn.v_proj.weight": "attn_v",
                "self_attn.o_proj.weight": "attn_o", "self_attn.q_norm.weight": "attn_q_norm", "self_attn.k_norm.weight": "attn_k_norm",
                "mlp.gate_proj.weight": "ffn_gate", "mlp.up_proj.weight": "ffn_up", "mlp.down_proj.weight": "ffn_down",
                "layer_scalar": "layer_scalar", "per_layer_input_gate.weight": "ple_gate", "per_layer_projection.weight": "ple_proj",
                "post_per_layer_input_norm.weight": "ple_post_norm", "router.proj.weight": "ffn_router", "router.scale": "ffn_router_scale",
                "router.per_expert_scale": "ffn_expert_scale", "experts.gate_up_proj": "experts_in", "experts.down_proj": "experts_out",
                "post_feedforward_layernorm_1.weight": "ffn_post_norm_1", "post_feedforward_layernorm_2.weight": "ffn_post_norm_2",
                "pre_feedforward_layernorm_2.weight": "ffn_norm_2"}


def _map_gemma4(cfg, store: WeightStore) -> Dict[str, PackedWeight]:
    """Gemma 4 text tensors (``model.*`` of a text checkpoint, ``model.language_model.*`` of a multimodal one).  The
    experts are stored stacked in the tracer's own layout; K/V projections of layers that share another layer's K/V
    are present in the file and unused."""
    canon: Dict[str, PackedWeight] = {}
    for n in store.names():
        m = re.match(r"model\.(?:language_model\.)?(.+)$", n)
        if n == "lm_head.weight":
            canon["lm_head"] = store[n]
        if not m:
            continue
        rest = m.group(1)
        if rest in GEMMA4_TOP:
            canon[GEMMA4_TOP[rest]] = store[n]
            continue
        lm = re.match(r"layers\.(\d+)\.(.+)$", rest)
        if lm and lm.group(2) in GEMMA4_LAYER:
            l, role = int(lm.group(1)), GEMMA4_LAYER[lm.group(2)]
            if role in ("attn_k", "attn_v", "attn_k_norm") and cfg.kv_source(l) is not None:
                continue
            if role == "attn_v" and cfg.value_is_key(l):
                continue
            canon[f"layers.{l}.{role}"] = store[n]
    return canon


QWEN_VISION_LAYER = {"norm1.weight": "attn_norm", "norm2.weight": "ffn_norm", "attn.proj.weight": "attn_o", "attn.proj.bias": "attn_o_bias",
                     "mlp.gate_proj.weight": "ffn_gate", "mlp.gate_proj.bias": "ffn_gate_bias", "mlp.up_proj.weight": "ffn_up",
                     "mlp.up_proj.bias": "ffn_up_bias", "mlp.down_proj.weight": "ffn_down", "mlp.down_proj.bias": "ffn_down_bias"}
QWEN_VISION_TOP = {"merger.ln_q.weight": "merger_norm", "merger.mlp.0.weight": "merger_fc1", "merger.mlp.0.bias": "merger_fc1_bias",
                   "merger.mlp.2.weight": "merger_fc2", "merger.mlp.2.bias": "merger_fc2_bias"}


def _map_qwen_vision(store: WeightStore) -> Dict[str, PackedWeight]:
    """Vision tower tensors of a Qwen2.5-VL checkpoint (``model.visual.*``, older files ``visual.*``): the patch
    convolution ``[out, C, t, p, p]`` flattens to a matrix, the fused ``qkv`` rows are cut into thirds."""
    canon: Dict[str, PackedWeight] = {}
    for n in store.names():
        m = re.match(r"(?:model\.)?visual\.(.+)$", n)
        if not m:
            continue
        short = m.group(1)
        if short == "patch_embed.proj.weight":
            w = store[n].to_f32()
            canon["vision.patch_embed"] = f32_weight("vision.patch_embed", w.reshape(w.shape[0], -1))
        elif short in QWEN_VISION_TOP:
            canon["vision." + QWEN_VISION_TOP[short]] = store[n]
        else:
            b = re.match(r"blocks\.(\d+)\.(.+)$", short)
            if not b:
                continue
            p, rest = f"vision.layers.{b.group(1)}.", b.group(2)
            if rest in QWEN_VISION_LAYER:
                canon[p + QWEN_VISION_LAYER[rest]] = store[n]
            elif rest in ("attn.qkv.weight", "attn.qkv.bias"):
                w = store[n].to_f32()
                third = w.shape[0] // 3
                tail = "_bias" if rest.endswith("bias") else ""
                for i, role in enumerate(("attn_q", "attn_k", "attn_v")):
                    canon[p + role + tail] = f32_weight(p + role + tail, np.ascontiguousarray(w[i * third:(i + 1) * third]))
    return canon


def map_checkpoint(cfg: DecoderConfig, store: WeightStore) -> Dict[str, PackedWeight]:
    """Canonical role name -> stored tensor for one Hugging Face checkpoint of ``cfg``'s family."""
    if cfg.family == "qwen_vl":
        text = replace(cfg, family="qwen2")
        return {**_map_qwen_vision(store), **map_checkpoint(text, store)}
    if cfg.family == "gemma4":
        return _map_gemma4(cfg, store)
    if cfg.family == "deepseek4":
        return _map_deepseek4(cfg, store)
    if cfg.family == "idefics3":
        text = replace(cfg, family="llama")
        return {**_map_vision(store), **map_checkpoint(text, _Renamed(store, "model.text_model.", "model."))}
    if cfg.family == "bert":
        return _map_bert(cfg, store)
    if cfg.family == "nemotron_h":
        return _map_nemotron_h(cfg, store)
    if cfg.family == "mpt":
        return _map_mpt(cfg, store)
    if cfg.family == "bloom":
        return _map_bloom(cfg, store)
    table = dict(LAYER)
    if cfg.block == "post":
        table.update(POST_BLOCK)
        table.pop("input_layernorm.weight")
    elif cfg.block == "sandwich":
        table.update(SANDWICH_BLOCK)
    canon: Dict[str, PackedWeight] = {}
    mx_parts: Dict[str, Dict[str, np.ndarray]] = {}       # gpt-oss: a layer's MXFP4 expert operands, assembled once all are seen
    names = store.names()
    for n in names:
        w = store[n]
        if n in TOP:
            canon[TOP[n]] = w
            continue
        m = re.match(r"model\.(?:language_model\.)?layers\.(\d+)\.(.+)$", n)
        if not m:
            top = re.match(r"model\.(?:language_model\.)?hyper_connection_mixer\.(.+)$", n) if cfg.hc_count else None
            if top and _qwen38_gate("hc_final_", top.group(1)):
                canon[_qwen38_gate("hc_final_", top.group(1))] = w
            continue
        l, rest = int(m.group(1)), m.group(2)
        p = f"layers.{l}."
        if cfg.family == "qwen38" and _qwen38_tensor(cfg, p, rest, w, canon):
            continue
        if cfg.family in ("qwen3next", "qwen38_27b", "qwen38") and _qwen3next_tensor(cfg, p, rest, w, canon):
            continue
        if cfg.family == "glm53_flash" and _glm53_tensor(cfg, l, p, rest, w, canon):
            continue
        if rest in table:
            canon[p + table[rest]] = w
            continue
        if l == cfg.n_layers and cfg.mtp_layers and rest in MTP:
            canon[MTP[rest]] = w
            continue
        e = re.match(r"(?:block_sparse_moe|mlp)\.experts\.(\d+)\.(\w+)\.weight$", rest)
        if e and e.group(2) in EXPERT:
            canon[p + f"experts.{e.group(1)}.{EXPERT[e.group(2)]}"] = w
            continue
        if rest == "self_attn.qkv_proj.weight":                       # Phi-3: q | k | v rows
            q, kv = cfg.q_size, cfg.kv_size
            if w.shape[0] != q + 2 * kv:
                raise CheckpointLayout(f"{n}: {w.shape[0]} rows, expected {q + 2 * kv} (q | k | v)")
            canon[p + "attn_q"], canon[p + "attn_k"], canon[p + "attn_v"] = w.rows(0, q), w.rows(q, kv), w.rows(q + kv, kv)
        elif rest == "mlp.gate_up_proj.weight":                       # Phi-3: gate | up rows
            half = w.shape[0] // 2
            if half != cfg.ffn:
                raise CheckpointLayout(f"{n}: {w.shape[0]} rows, expected {2 * cfg.ffn} (gate | up)")
            canon[p + "ffn_gate"], canon[p + "ffn_up"] = w.rows(0, half), w.rows(half, half)
        elif cfg.family == "gpt_oss" and rest[len("mlp.experts."):] in MX_PARTS and rest.startswith("mlp.experts."):
            raw = w.planar.get("__raw__") if w.planar else None
            if raw is None:
                raise CheckpointLayout(f"{n}: MXFP4 operands are stored as bytes, found {w.format}")
            mx_parts.setdefault(p, {})[rest[len("mlp.experts."):]] = raw
        elif cfg.family == "gpt_oss" and rest.startswith("mlp.experts."):
            _gpt_oss_experts(cfg, p, rest, w, canon)
        elif rest in ("mlp.experts.gate_up_proj", "block_sparse_moe.input_linear.weight"):   # stacked [E, 2F, H]
            F = cfg.moe_ffn
            if tuple(w.shape) != (cfg.n_experts, 2 * F, cfg.hidden):
                raise CheckpointLayout(f"{n}: shape {w.shape}, expected {(cfg.n_experts, 2 * F, cfg.hidden)}")
            for x in range(cfg.n_experts):
                gu = first_axis(w, x)
                canon[p + f"experts.{x}.gate"], canon[p + f"experts.{x}.up"] = gu.rows(0, F), gu.rows(F, F)
        elif rest in ("mlp.experts.down_proj", "block_sparse_moe.output_linear.weight"):     # stacked [E, H, F]
            for x in range(cfg.n_experts):
                canon[p + f"experts.{x}.down"] = first_axis(w, x)
    for p, parts in mx_parts.items():
        _gpt_oss_mxfp4(cfg, p, parts, canon)
    if cfg.family == "qwen38":
        _join_table_shards(canon)
    if cfg.norm_offset != 0.0:
        for k in list(canon):
            if k.endswith("norm"):
                canon[k] = f32_weight(k, canon[k].to_f32() + cfg.norm_offset)
    if cfg.rope_interleaved and cfg.is_mla:
        _mla_halfsplit(cfg, canon)
    return canon


def _qwen3next_tensor(cfg: DecoderConfig, p: str, rest: str, w: PackedWeight, canon: Dict[str, PackedWeight]) -> bool:
    """Tensors of the gated attention and gated delta-net layers that are stored fused (crates/poot-models/src/
    architectures/qwen3next.rs): ``q_proj`` carries ``[head][query | gate]`` rows; ``in_proj_qkvz`` is grouped per key
    head as ``[q | k | v of the group's value heads | z of them]`` and ``in_proj_ba`` as ``[b | a]``."""
    nk, nv, Dg, D = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.head_dim
    if rest == "self_attn.q_proj.weight":
        a = w.to_f32().reshape(cfg.n_heads, 2, D, -1)
        canon[p + "attn_q"] = f32_weight(p + "attn_q", a[:, 0].reshape(cfg.n_heads * D, -1))
        canon[p + "attn_gate"] = f32_weight(p + "attn_gate", a[:, 1].reshape(cfg.n_heads * D, -1))
        return True
    if rest == "linear_attn.in_proj_qkvz.weight":
        r = nv // nk
        a = w.to_f32().reshape(nk, 2 * Dg + 2 * r * Dg, -1)
        cuts = {"gdn_q": (0, Dg), "gdn_k": (Dg, Dg), "gdn_v": (2 * Dg, r * Dg), "gdn_z": (2 * Dg + r * Dg, r * Dg)}
        for role, (o, n) in cuts.items():
            canon[p + role] = f32_weight(p + role, a[:, o:o + n].reshape(nk * n, -1))
        return True
    if rest == "linear_attn.in_proj_ba.weight":
        r = nv // nk
        a = w.to_f32().reshape(nk, 2 * r, -1)
        canon[p + "gdn_b"] = f32_weight(p + "gdn_b", a[:, :r].reshape(nv, -1))
        canon[p + "gdn_a"] = f32_weight(p + "gdn_a", a[:, r:].reshape(nv, -1))
        return True
    if rest == "linear_attn.in_proj_qkv.weight":        # Qwen3.5 spelling: q | k | v rows, one projection per quantity
        kd = nk * Dg
        canon[p + "gdn_q"], canon[p + "gdn_k"], canon[p + "gdn_v"] = w.rows(0, kd), w.rows(kd, kd), w.rows(2 * kd, nv * Dg)
        return True
    simple = {"linear_attn.in_proj_z.weight": "gdn_z", "linear_attn.in_proj_b.weight": "gdn_b", "linear_attn.in_proj_a.weight": "gdn_a",
              "linear_attn.dt_bias": "gdn_dt_bias", "linear_attn.A_log": "gdn_a_log", "linear_attn.norm.weight": "gdn_gate_norm_w",
              "linear_attn.out_proj.weight": "gdn_o"}
    if rest in simple:
        canon[p + simple[rest]] = w
        return True
    if rest == "linear_attn.conv1d.weight":                # [C, 1, K]
        a = w.to_f32()
        canon[p + "gdn_conv"] = f32_weight(p + "gdn_conv", a.reshape(a.shape[0], a.shape[-1]))
        return True
    return False


def qwen35_gguf_tensor(cfg: DecoderConfig, p: str, rest: str, w: PackedWeight, canon: Dict[str, PackedWeight]) -> bool:
    """llama.cpp's spelling of a Qwen3.5 layer (``general.architecture = qwen35``; crates/poot-models/src/architectures/
    qwen38_27b.rs:19-23): one tensor per delta-net quantity (``attn_qkv`` = q | k | v rows, ``attn_gate`` = z, ``ssm_beta``,
    ``ssm_alpha``), the value heads tiled over the key heads instead of grouped, ``ssm_a`` already ``-exp(A_log)``, the conv
    kernel as ``[channels, taps]``; the attention layers' ``attn_q`` carries ``[head][query | gate]`` rows as the source does."""
    from .names import gdn_grouped_heads
    nk, nv, Dg, D = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.head_dim
    kd = nk * Dg
    grouped = gdn_grouped_heads(nv, nk) if nk else None

    def untile(a: np.ndarray, block: int) -> np.ndarray:
        """Rows of ``a`` in runs of ``block`` per value head, put back from tiled to grouped order."""
        t = a.reshape(nv, block, -1)
        out = np.empty_like(t)
        out[grouped] = t
        return out.reshape(a.shape)

    if rest == "attn_q.weight" and w.shape[0] == 2 * cfg.n_heads * D:
        a = w.to_f32().reshape(cfg.n_heads, 2, D, -1)
        canon[p + "attn_q"] = f32_weight(p + "attn_q", a[:, 0].reshape(cfg.n_heads * D, -1))
        canon[p + "attn_gate"] = f32_weight(p + "attn_gate", a[:, 1].reshape(cfg.n_heads * D, -1))
        return True
    if rest == "attn_qkv.weight":
        if w.shape[0] != 2 * kd + nv * Dg:
            raise CheckpointLayout(f"{p}{rest}: {w.shape[0]} rows, expected {2 * kd + nv * Dg}")
        canon[p + "gdn_q"], canon[p + "gdn_k"] = w.rows(0, kd), w.rows(kd, kd)
        canon[p + "gdn_v"] = f32_weight(p + "gdn_v", untile(w.rows(2 * kd, nv * Dg).to_f32(), Dg))
        return True
    per_head = {"attn_gate.weight": ("gdn_z", Dg), "ssm_beta.weight": ("gdn_b", 1), "ssm_alpha.weight": ("gdn_a", 1), "ssm_dt.bias": ("gdn_dt_bias", 1)}
    if rest in per_head:
        role, block = per_head[rest]
        canon[p + role] = f32_weight(p + role, untile(w.to_f32(), block))
        return True
    if rest == "ssm_a":
        a = w.to_f32()
        if not (a < 0).all():
            raise CheckpointLayout(f"{p}ssm_a holds -exp(A_log): every value is negative")
        canon[p + "gdn_a_log"] = f32_weight(p + "gdn_a_log", untile(np.log(-a.astype(np.float64)).astype(np.float32), 1))
        return True
    if rest == "ssm_conv1d.weight":
        a = w.to_f32().reshape(2 * kd + nv * Dg, -1)
        canon[p + "gdn_conv"] = f32_weight(p + "gdn_conv", np.concatenate([a[:2 * kd], untile(a[2 * kd:], Dg)], 0))
        return True
    if rest == "ssm_out.weight":                           # [hidden, value channels]: the columns follow the value heads
        a = w.to_f32()
        canon[p + "gdn_o"] = f32_weight(p + "gdn_o", np.ascontiguousarray(untile(np.ascontiguousarray(a.T), Dg).T))
        return True
    return False


GLM53_SITE = {f"hc_{site}_{part}": f"hc_{site}_{part}" for site in ("attn", "ffn") for part in ("fn", "base", "scale")}
GLM53_KDA = {"self_attn.q_proj.weight": "kda_q", "self_attn.k_proj.weight": "kda_k", "self_attn.v_proj.weight": "kda_v",
             "self_attn.f_a_proj.weight": "kda_f_a", "self_attn.f_b_proj.weight": "kda_f_b", "self_attn.b_proj.weight": "kda_b",
             "self_attn.g_a_proj.weight": "kda_g_a", "self_attn.g_b_proj.weight": "kda_g_b", "self_attn.A_log": "kda_a_log",
             "self_attn.dt_bias": "kda_dt_bias", "self_attn.o_norm.weight": "kda_o_norm", "self_attn.o_proj.weight": "kda_o"}
GLM53_POOL = {"self_attn.indexer.index_kpool_compress_gate": "idx_pool_gate", "self_attn.indexer.index_kpool_compress_ape": "idx_pool_bias"}


def _glm53_tensor(cfg, l: int, p: str, rest: str, w: PackedWeight, canon: Dict[str, PackedWeight]) -> bool:
    """Tensors GLM-5.3-Flash names its own way (crates/poot-models/src/architectures/glm53_flash/names.rs): the
    hyper-connection sites, the delta-attention layer (whose projections share names with attention's) and the pooling
    of the indexer.  The layer after the text stack is the multi-token-prediction block: latent attention."""
    if rest in GLM53_SITE:
        canon[p + GLM53_SITE[rest]] = w
        return True
    if rest in GLM53_POOL:
        canon[p + GLM53_POOL[rest]] = w
        return True
    if l < cfg.n_layers and cfg.mixer_of(l) == "kda":
        if rest in GLM53_KDA:
            canon[p + GLM53_KDA[rest]] = w
            return True
        m = re.match(r"self_attn\.([qkv])_conv1d\.weight$", rest)
        if m:                                            # [C, 1, K]
            a = w.to_f32()
            canon[p + "kda_conv_" + m.group(1)] = f32_weight(p + "kda_conv_" + m.group(1), a.reshape(a.shape[0], a.shape[-1]))
            return True
    return False


DEEPSEEK4_TOP = {"embed.weight": "embed", "norm.weight": "final_norm", "head.weight": "lm_head", "hc_head_fn": "hc_head_fn",
                 "hc_head_base": "hc_head_base", "hc_head_scale": "hc_head_scale"}
DEEPSEEK4_LAYER = {
    "attn_norm.weight": "attn_norm", "ffn_norm.weight": "ffn_norm", "attn.q_norm.weight": "attn_q_a_norm",
    "attn.kv_norm.weight": "attn_kv_norm", "attn.attn_sink": "attn_sinks", "attn.wq_a.weight": "attn_q_a", "attn.wq_b.weight": "attn_q_b",
    "attn.wkv.weight": "attn_kv", "attn.wo_a.weight": "attn_o_a", "attn.wo_b.weight": "attn_o", "ffn.gate.weight": "ffn_router",
    "ffn.gate.bias": "ffn_router_select_bias", "ffn.shared_experts.w1.weight": "shared_gate", "ffn.shared_experts.w3.weight": "shared_up",
    "ffn.shared_experts.w2.weight": "shared_down", "attn.compressor.wkv.weight": "cmp_kv", "attn.compressor.wgate.weight": "cmp_gate",
    "attn.compressor.ape": "cmp_bias", "attn.compressor.norm.weight": "cmp_norm", "attn.indexer.wq_b.weight": "idx_q",
    "attn.indexer.weights_proj.weight": "idx_weights", "attn.indexer.compressor.wkv.weight": "idx_cmp_kv",
    "attn.indexer.compressor.wgate.weight": "idx_cmp_gate", "attn.indexer.compressor.ape": "idx_cmp_bias",
    "attn.indexer.compressor.norm.weight": "idx_cmp_norm",
    **{f"hc_{site}_{part}": f"hc_{site}_{part}" for site in ("attn", "ffn") for part in ("fn", "base", "scale")}}


def _map_deepseek4(cfg, store: WeightStore) -> Dict[str, PackedWeight]:
    """DeepSeek-V4 tensors in the release's own naming (no ``model.`` prefix: ``embed.weight``, ``layers.N.attn.wq_a.weight``,
    ``layers.N.ffn.experts.E.w1.weight``, ``head.weight``; crates/poot-models/src/architectures/deepseek4/names.rs).  A
    hash-routed layer's token-to-experts table (``ffn.gate.tid2eid``, integers) is kept as exact small numbers."""
    canon: Dict[str, PackedWeight] = {}
    for n in store.names():
        if n in DEEPSEEK4_TOP:
            canon[DEEPSEEK4_TOP[n]] = store[n]
            continue
        m = re.match(r"layers\.(\d+)\.(.+)$", n)
        if not m:
            continue
        p, rest = f"layers.{m.group(1)}.", m.group(2)
        if rest in DEEPSEEK4_LAYER:
            canon[p + DEEPSEEK4_LAYER[rest]] = store[n]
        elif rest == "ffn.gate.tid2eid":
            w = store[n]
            raw = w.planar["__raw__"] if getattr(w, "planar", None) and "__raw__" in w.planar else w.to_f32()
            if raw.min() < 0 or raw.max() >= cfg.n_experts:
                raise CheckpointLayout(f"{n}: expert ids outside [0, {cfg.n_experts})")
            canon[p + "ffn_hash_table"] = f32_weight(p + "ffn_hash_table", np.asarray(raw, np.float32))
        else:
            e = re.match(r"ffn\.experts\.(\d+)\.(w[123])\.weight$", rest)
            if e:
                canon[p + f"experts.{e.group(1)}.{EXPERT[e.group(2)]}"] = store[n]
    return canon


QWEN38_GATE = {"hc_norm.weight": "norm", "input_mix_weight_down": "down", "input_mix_weight_up": "up", "block_inject_weight": "inject"}
QWEN38_PLE = {"ple.ple_embedding.ngram_embedding.weight": "ple_table", "ple.key_proj.weight": "ple_key", "ple.value_proj.weight": "ple_value",
              "ple.norm_key.weight": "ple_key_norm", "ple.norm_query.weight": "ple_query_norm", "ple.norm_conv.weight": "ple_conv_norm"}


def _qwen38_gate(stem: str, rest: str):
    """``<gate>.<tensor>[.weight]`` of a hyper-connection gate -> canonical suffix."""
    rest = rest[:-len(".weight")] if rest.endswith(".weight") and rest != "hc_norm.weight" else rest
    return stem + QWEN38_GATE[rest] if rest in QWEN38_GATE else None


def _join_table_shards(canon: Dict[str, PackedWeight]) -> None:
    """An n-gram table stored as ``shard_0, shard_1, ...`` (consecutive row ranges of E4M3 codes) with one ``weight_scale``
    becomes one table that stays at a byte per value: fp8 codes with the scale repeated per row, which is the
    per-channel fp8 format the row gather already reads.  The reference keeps the shards apart and selects among one
    gather per shard because a single buffer of its devices cannot hold the table (crates/poot-models/src/components/
    ple.rs:24-28); one allocation of this device can."""
    stems = sorted({k.split("#")[0] for k in canon if "ple_table#" in k})
    for stem in stems:
        parts = {k.split("#")[1]: canon.pop(k) for k in [k for k in canon if k.startswith(stem + "#")]}
        scale = parts.pop("scale", None)
        if scale is None:
            raise CheckpointLayout(f"{stem}: table shards without their weight_scale")
        order = sorted(parts, key=int)
        if order != [str(i) for i in range(len(order))]:
            raise CheckpointLayout(f"{stem}: shards {order} do not count up from 0")
        codes = []
        for i in order:
            w = parts[i]
            raw = (w.planar or {}).get("__raw__")
            if raw is None or raw.dtype.itemsize != 1 or raw.ndim != 2:
                raise CheckpointLayout(f"{stem}.shard_{i}: expected a matrix of fp8 codes")
            if codes and raw.shape[1] != codes[0].shape[1]:
                raise CheckpointLayout(f"{stem}.shard_{i}: {raw.shape[1]} columns, the first shard has {codes[0].shape[1]}")
            codes.append(raw.view(np.uint8))
        sraw = (scale.planar or {}).get("__raw__")
        sval = np.asarray(sraw if sraw is not None else scale.to_f32(), np.float32).reshape(-1)
        if sval.size != 1:
            raise CheckpointLayout(f"{stem}: one scale for the whole table, got {sval.size}")
        table = np.concatenate(codes, 0)
        canon[stem] = PackedWeight(stem, "E4M3_CHANNEL", tuple(table.shape), np.zeros(0, np.uint8),
                                   planar={"weight": table, "weight_scale": np.full(table.shape[0], sval[0], np.float32)})


def _qwen38_tensor(cfg, p: str, rest: str, w: PackedWeight, canon: Dict[str, PackedWeight]) -> bool:
    """Tensors Qwen3.8-Flash-Next adds to the Qwen3.5 layer (crates/poot-models/src/architectures/qwen38/config.rs): the
    two hyper-connection gates, the n-gram embedding block and the block indexer, whose query rows and key rows are
    one fused projection, query rows first."""
    for site, stem in (("attn_hyper_connection.", "hc_attn_"), ("mlp_hyper_connection.", "hc_ffn_")):
        if rest.startswith(site):
            name = _qwen38_gate(p + stem, rest[len(site):])
            if name is not None:
                canon[name] = w
                return True
    if rest in QWEN38_PLE:
        canon[p + QWEN38_PLE[rest]] = w
        return True
    sh = re.match(r"ple\.ple_embedding\.ngram_embedding\.(?:shard_(\d+)\.weight|(weight_scale))$", rest)
    if sh:                                                 # the table as numbered E4M3 row-range shards under one scale
        canon[p + ("ple_table#scale" if sh.group(2) else f"ple_table#{int(sh.group(1))}")] = w
        return True
    if rest == "ple.conv1d.weight":                        # [C, 1, K]
        a = w.to_f32()
        canon[p + "ple_conv"] = f32_weight(p + "ple_conv", a.reshape(a.shape[0], a.shape[-1]))
        return True
    if rest == "self_attn.indexer.index_qk_proj.weight":
        nq = cfg.index_n_heads * cfg.index_head_dim
        if w.shape[0] != nq + cfg.index_head_dim:
            raise CheckpointLayout(f"{w.name}: {w.shape[0]} rows, expected {nq + cfg.index_head_dim} (queries | key)")
        canon[p + "idx_q"], canon[p + "idx_k"] = w.rows(0, nq), w.rows(nq, cfg.index_head_dim)
        return True
    if rest in ("self_attn.indexer.q_layernorm.weight", "self_attn.indexer.k_layernorm.weight"):
        canon[p + ("idx_q_norm" if ".q_" in rest else "idx_k_norm")] = w
        return True
    return False


NEMOTRON_MIXER = {"mixer.dt_bias": "ssm_dt_bias", "mixer.A_log": "ssm_a_log", "mixer.D": "ssm_d", "mixer.conv1d.bias": "ssm_conv_bias",
                  "mixer.norm.weight": "ssm_gate_norm_w", "mixer.out_proj.weight": "ssm_o",
                  "mixer.q_proj.weight": "attn_q", "mixer.k_proj.weight": "attn_k", "mixer.v_proj.weight": "attn_v",
                  "mixer.o_proj.weight": "attn_o", "mixer.up_proj.weight": "ffn_up", "mixer.down_proj.weight": "ffn_down",
                  "mixer.gate.weight": "ffn_router", "mixer.gate.e_score_correction_bias": "ffn_router_select_bias",
                  "mixer.shared_experts.up_proj.weight": "shared_up", "mixer.shared_experts.down_proj.weight": "shared_down"}


def _map_nemotron_h(cfg: DecoderConfig, store: WeightStore) -> Dict[str, PackedWeight]:
    canon: Dict[str, PackedWeight] = {}
    I = cfg.ssm_heads * cfg.ssm_head_dim
    C = I + 2 * cfg.ssm_groups * cfg.ssm_state
    top = {"embeddings.weight": "embed", "embedding.weight": "embed", "norm_f.weight": "final_norm"}
    for n in store.names():
        w = store[n]
        if n == "lm_head.weight":
            canon["lm_head"] = w
            continue
        short = re.sub(r"^(model|backbone)\.", "", n)
        if short in top:
            canon[top[short]] = w
            continue
        m = re.match(r"layers\.(\d+)\.(.+)$", short)
        if not m:
            continue
        l, rest = int(m.group(1)), m.group(2)
        p = f"layers.{l}."
        if rest == "norm.weight":          # one norm per block: it feeds the block's mixer, or its FFN when it has none
            canon[p + ("attn_norm" if cfg.mixer_of(l) != "none" else "ffn_norm")] = w
        elif rest in NEMOTRON_MIXER:
            canon[p + NEMOTRON_MIXER[rest]] = w
        elif rest == "mixer.in_proj.weight":               # z | (x | B | C) | dt rows
            if w.shape[0] != I + C + cfg.ssm_heads:
                raise CheckpointLayout(f"{n}: {w.shape[0]} rows, expected {I + C + cfg.ssm_heads}")
            canon[p + "ssm_in_z"], canon[p + "ssm_in_x"], canon[p + "ssm_in_dt"] = w.rows(0, I), w.rows(I, C), w.rows(I + C, cfg.ssm_heads)
        elif rest == "mixer.conv1d.weight":
            a = w.to_f32()
            canon[p + "ssm_conv"] = f32_weight(p + "ssm_conv", a.reshape(a.shape[0], a.shape[-1]))
        elif re.match(r"mixer\.experts\.(\d+)\.(up|down)_proj\.weight$", rest):
            e = re.match(r"mixer\.experts\.(\d+)\.(up|down)_proj\.weight$", rest)
            canon[p + f"experts.{e.group(1)}.{e.group(2)}"] = w
        elif rest == "mixer.experts.up_proj":
            for x in range(cfg.n_experts):
                canon[p + f"experts.{x}.up"] = first_axis(w, x)
        elif rest == "mixer.experts.down_proj":
            for x in range(cfg.n_experts):
                canon[p + f"experts.{x}.down"] = first_axis(w, x)
    return canon


def _gpt_oss_experts(cfg: DecoderConfig, p: str, rest: str, w: PackedWeight, canon: Dict[str, PackedWeight]) -> None:
    E, F = cfg.n_experts, cfg.moe_ffn
    a = w.to_f32()
    if rest == "mlp.experts.gate_up_proj":                 # [E, H, 2F], gate at even columns, up at odd ones
        for x in range(E):
            canon[p + f"experts.{x}.gate"] = f32_weight(f"{p}experts.{x}.gate", a[x][:, 0::2].T)
            canon[p + f"experts.{x}.up"] = f32_weight(f"{p}experts.{x}.up", a[x][:, 1::2].T)
    elif rest == "mlp.experts.gate_up_proj_bias":          # [E, 2F] alternating
        canon[p + "experts_in_bias"] = f32_weight(p + "experts_in_bias", np.concatenate([a[:, 0::2], a[:, 1::2]], 1))
    elif rest == "mlp.experts.down_proj":                  # [E, F, H]
        for x in range(E):
            canon[p + f"experts.{x}.down"] = f32_weight(f"{p}experts.{x}.down", a[x].T)
    elif rest == "mlp.experts.down_proj_bias":
        canon[p + "experts_out_bias"] = f32_weight(p + "experts_out_bias", a)


MX_PARTS = ("gate_up_proj_blocks", "gate_up_proj_scales", "down_proj_blocks", "down_proj_scales")


def _gpt_oss_mxfp4(cfg: DecoderConfig, p: str, parts: Dict[str, np.ndarray], canon: Dict[str, PackedWeight]) -> None:
    """The released gpt-oss checkpoints store the experts as MXFP4: ``*_blocks[E, rows, K / 32, 16]`` bytes of two 4-bit
    E2M1 codes each (even element in the low nibble) and ``*_scales[E, rows, K / 32]`` E8M0 exponents, one per 32 values.
    That is the planar ``E2M1_ROW32`` format row for row, so every expert becomes a packed weight without decoding a
    value: gate rows are the even rows of ``gate_up``, up rows the odd ones; ``down`` is ``[H, F]`` as stored
    (crates/poot-models/src/architectures/gpt_oss.rs)."""
    missing = [k for k in MX_PARTS if k not in parts]
    if missing:
        raise CheckpointLayout(f"{p}mlp.experts: MXFP4 experts without {', '.join(missing)}")
    E, F, H = cfg.n_experts, cfg.moe_ffn, cfg.hidden
    for stem, rows, K in (("gate_up_proj", 2 * F, H), ("down_proj", H, F)):
        blocks, scales = parts[stem + "_blocks"], parts[stem + "_scales"]
        if blocks.dtype != np.uint8 or scales.dtype != np.uint8 or K % 32:
            raise CheckpointLayout(f"{p}mlp.experts.{stem}: MXFP4 operands are bytes over rows of whole 32-value blocks")
        if tuple(blocks.shape) != (E, rows, K // 32, 16) or tuple(scales.shape) != (E, rows, K // 32):
            raise CheckpointLayout(f"{p}mlp.experts.{stem}: blocks {tuple(blocks.shape)} / scales {tuple(scales.shape)}, expected "
                                   f"{(E, rows, K // 32, 16)} / {(E, rows, K // 32)}")
    gu_b, gu_s = parts["gate_up_proj_blocks"].reshape(E, 2 * F, H // 2), parts["gate_up_proj_scales"]
    dn_b, dn_s = parts["down_proj_blocks"].reshape(E, H, F // 2), parts["down_proj_scales"]
    packed = lambda name, n, k, wt, sc: PackedWeight(name, "E2M1_ROW32", (n, k), np.zeros(0, np.uint8),
                                                      planar={"weight": np.ascontiguousarray(wt), "weight_scale": np.ascontiguousarray(sc)})
    for x in range(E):
        canon[p + f"experts.{x}.gate"] = packed(f"{p}experts.{x}.gate", F, H, gu_b[x, 0::2], gu_s[x, 0::2])
        canon[p + f"experts.{x}.up"] = packed(f"{p}experts.{x}.up", F, H, gu_b[x, 1::2], gu_s[x, 1::2])
        canon[p + f"experts.{x}.down"] = packed(f"{p}experts.{x}.down", H, F, dn_b[x], dn_s[x])


def _mla_halfsplit(cfg: DecoderConfig, canon: Dict[str, PackedWeight]) -> None:
    dn, dr, nh = cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.n_heads
    perm = _deinterleave_rows(dr)
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        qn = p + ("attn_q_b" if cfg.q_lora_rank else "attn_q")
        q = canon[qn].to_f32().reshape(nh, dn + dr, -1)
        q = np.concatenate([q[:, :dn], q[:, dn:][:, perm]], 1).reshape(nh * (dn + dr), -1)
        canon[qn] = f32_weight(qn, q)
        kv = canon[p + "attn_kv_a"].to_f32()
        kv = np.concatenate([kv[:cfg.kv_lora_rank], kv[cfg.kv_lora_rank:][perm]], 0)
        canon[p + "attn_kv_a"] = f32_weight(p + "attn_kv_a", kv)


def _map_mpt(cfg: DecoderConfig, store: WeightStore) -> Dict[str, PackedWeight]:
    canon: Dict[str, PackedWeight] = {}
    for n in store.names():
        w = store[n]
        if n == "transformer.wte.weight":
            canon["embed"] = w
        elif n == "transformer.norm_f.weight":
            canon["final_norm"] = w
        elif n == "lm_head.weight":
            canon["lm_head"] = w
        else:
            m = re.match(r"transformer\.blocks\.(\d+)\.(.+)$", n)
            if not m:
                continue
            p, rest = f"layers.{m.group(1)}.", m.group(2)
            if rest in MPT_LAYER:
                canon[p + MPT_LAYER[rest]] = w
            elif rest == "attn.Wqkv.weight":               # q | k | v thirds
                H = cfg.hidden
                if w.shape[0] != 3 * H:
                    raise CheckpointLayout(f"{n}: {w.shape[0]} rows, expected {3 * H}")
                canon[p + "attn_q"], canon[p + "attn_k"], canon[p + "attn_v"] = w.rows(0, H), w.rows(H, H), w.rows(2 * H, H)
    return canon


def _map_bloom(cfg: DecoderConfig, store: WeightStore) -> Dict[str, PackedWeight]:
    canon: Dict[str, PackedWeight] = {}
    nh, D = cfg.n_heads, cfg.head_dim
    for n in store.names():
        w = store[n]
        if n in BLOOM_TOP:
            canon[BLOOM_TOP[n]] = w
            continue
        m = re.match(r"transformer\.h\.(\d+)\.(.+)$", n)
        if not m:
            continue
        p, rest = f"layers.{m.group(1)}.", m.group(2)
        if rest in BLOOM_LAYER:
            canon[p + BLOOM_LAYER[rest]] = w
        elif rest == "self_attention.query_key_value.weight":      # rows ordered [head][q|k|v][channel]
            a = w.to_f32().reshape(nh, 3, D, -1)
            for i, role in enumerate(("attn_q", "attn_k", "attn_v")):
                canon[p + role] = f32_weight(p + role, a[:, i].reshape(nh * D, -1))
        elif rest == "self_attention.query_key_value.bias":
            a = w.to_f32().reshape(nh, 3, D)
            for i, role in enumerate(("attn_q_bias", "attn_k_bias", "attn_v_bias")):
                canon[p + role] = f32_weight(p + role, a[:, i].reshape(nh * D))
    return canon
