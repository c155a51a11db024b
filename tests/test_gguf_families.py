"""GGUF checkpoints of the families beyond llama / qwen: a Hugging Face model is written out the way llama.cpp's
converter lays a GGUF out (tensor names, Q / K rows permuted for the interleaved-rotary families, Gemma norm scales with
the one folded in, experts stacked ``[E, out, in]``, gpt-oss's norm names, sinks and per-expert biases), loaded by its
``general.architecture`` and evaluated: logits equal the Hugging Face forward."""
import re

import numpy as np
import pytest
import torch

from poot_b200.driver.handle import ModelHandle
from poot_b200.load import gguf, names
from poot_b200.models.model import StepSpec
from poot_b200.oracle.runner import OracleSession
from poot_b200.quant import codec
from poot_b200.quant.weights import PackedWeight
from tests.test_hf_parity import BASE, CASES, build

ARCH = {"olmo2": "olmo2", "olmoe": "olmoe", "smollm3": "smollm3", "granite": "granite", "granitemoe": "granitemoe", "gemma2": "gemma2",
        "gemma3": "gemma3", "gpt_oss": "gpt-oss"}
LAYER = {"input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
         "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
         "self_attn.o_proj.weight": "attn_output.weight", "self_attn.q_norm.weight": "attn_q_norm.weight",
         "self_attn.k_norm.weight": "attn_k_norm.weight", "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
         "mlp.down_proj.weight": "ffn_down.weight", "self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.bias": "attn_k.bias",
         "self_attn.v_proj.bias": "attn_v.bias", "self_attn.o_proj.bias": "attn_output.bias", "self_attn.sinks": "attn_sinks.weight",
         "mlp.gate.weight": "ffn_gate_inp.weight", "mlp.router.weight": "ffn_gate_inp.weight", "mlp.router.bias": "ffn_gate_inp.bias",
         "block_sparse_moe.router.layer.weight": "ffn_gate_inp.weight"}
PER_FAMILY = {
    "olmo2": {"post_attention_layernorm.weight": "post_attention_norm.weight", "post_feedforward_layernorm.weight": "post_ffw_norm.weight"},
    "gemma": {"post_attention_layernorm.weight": "post_attention_norm.weight", "pre_feedforward_layernorm.weight": "ffn_norm.weight",
              "post_feedforward_layernorm.weight": "post_ffw_norm.weight"},
    "gpt_oss": {"post_attention_layernorm.weight": "post_attention_norm.weight"},
}


def _f32(name, a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return PackedWeight(name, "F32", tuple(a.shape), a.view(np.uint8).reshape(-1))


def _to_gguf(path, family, m, quantise=None):
    """llama.cpp's layout of the Hugging Face model ``m``."""
    c = m.config
    arch = ARCH[family]
    nh, nkv = c.num_attention_heads, c.num_key_value_heads
    meta = {"general.architecture": arch, "general.name": family, f"{arch}.block_count": c.num_hidden_layers,
            f"{arch}.embedding_length": c.hidden_size, f"{arch}.attention.head_count": nh, f"{arch}.attention.head_count_kv": nkv,
            f"{arch}.feed_forward_length": c.intermediate_size, f"{arch}.attention.key_length": c.head_dim,
            f"{arch}.rope.freq_base": float(getattr(c, "rope_theta", None) or (c.rope_parameters.get("rope_theta") if "rope_theta" in c.rope_parameters
                                                                               else c.rope_parameters["full_attention"]["rope_theta"])),
            f"{arch}.attention.layer_norm_rms_epsilon": float(c.rms_norm_eps), f"{arch}.context_length": c.max_position_embeddings,
            f"{arch}.vocab_size": c.vocab_size, "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2}
    experts = getattr(c, "num_local_experts", None) or getattr(c, "num_experts", None)
    if experts:
        meta[f"{arch}.expert_count"], meta[f"{arch}.expert_used_count"] = int(experts), int(c.num_experts_per_tok)
    if family.startswith("gemma"):
        meta[f"{arch}.attention.sliding_window"] = int(c.sliding_window)
        if family == "gemma2":
            meta[f"{arch}.attn_logit_softcapping"], meta[f"{arch}.final_logit_softcapping"] = float(c.attn_logit_softcapping), float(c.final_logit_softcapping)
        else:
            meta[f"{arch}.rope.freq_base_swa"] = float(c.rope_parameters["sliding_attention"]["rope_theta"])
    if family == "gpt_oss":
        meta[f"{arch}.attention.sliding_window"] = int(c.sliding_window)
    if family.startswith("granite"):
        meta.update({f"{arch}.embedding_scale": float(c.embedding_multiplier), f"{arch}.residual_scale": float(c.residual_multiplier),
                     f"{arch}.logit_scale": float(c.logits_scaling), f"{arch}.attention.scale": float(c.attention_multiplier)})
    paired = family == "smollm3"
    gemma = family.startswith("gemma")
    table = {**LAYER, **PER_FAMILY.get("gemma" if gemma else family, {})}
    tensors = []
    sd = {k: v.detach().float().numpy() for k, v in m.state_dict().items()}

    def put(name, a):
        if quantise and a.ndim == 2 and name.endswith(".weight") and "norm" not in name and a.shape[1] % 32 == 0 and "inp" not in name:
            tensors.append(PackedWeight(name, quantise, tuple(a.shape), codec.quantize(quantise, np.ascontiguousarray(a, dtype=np.float32))))
        else:
            tensors.append(_f32(name, a))

    for k, a in sd.items():
        if k == "model.embed_tokens.weight":
            put("token_embd.weight", a)
        elif k == "model.norm.weight":
            put("output_norm.weight", a + 1.0 if gemma else a)
        elif k == "lm_head.weight":
            if not getattr(c, "tie_word_embeddings", False):
                put("output.weight", a)
        else:
            mm = re.match(r"model\.layers\.(\d+)\.(.+)$", k)
            if not mm:
                continue
            b, rest = f"blk.{mm.group(1)}.", mm.group(2)
            if rest in table:
                if gemma and "norm" in rest:
                    a = a + 1.0                                   # the converter folds the one in
                if paired and rest in ("self_attn.q_proj.weight", "self_attn.k_proj.weight"):
                    a = a[names.hf_to_gguf_qk_row_order(a.shape[0], nh if "q_proj" in rest else nkv)]
                put(b + table[rest], a)
            elif rest == "mlp.experts.gate_up_proj" and family == "gpt_oss":          # [E, H, 2F], gate / up columns alternating
                put(b + "ffn_gate_exps.weight", a[:, :, 0::2].transpose(0, 2, 1))
                put(b + "ffn_up_exps.weight", a[:, :, 1::2].transpose(0, 2, 1))
            elif rest == "mlp.experts.gate_up_proj_bias":
                put(b + "ffn_gate_exps.bias", a[:, 0::2]); put(b + "ffn_up_exps.bias", a[:, 1::2])
            elif rest == "mlp.experts.down_proj" and family == "gpt_oss":             # [E, F, H]
                put(b + "ffn_down_exps.weight", a.transpose(0, 2, 1))
            elif rest == "mlp.experts.down_proj_bias":
                put(b + "ffn_down_exps.bias", a)
            elif rest == "mlp.experts.gate_up_proj":                                  # stacked [E, 2F, H]: gate rows, then up rows
                F = a.shape[1] // 2
                put(b + "ffn_gate_exps.weight", a[:, :F]); put(b + "ffn_up_exps.weight", a[:, F:])
            elif rest == "mlp.experts.down_proj":                                     # stacked [E, H, F]
                put(b + "ffn_down_exps.weight", a)
            elif rest == "block_sparse_moe.input_linear.weight":                      # granitemoe: [E, 2F, H]
                F = a.shape[1] // 2
                put(b + "ffn_gate_exps.weight", a[:, :F]); put(b + "ffn_up_exps.weight", a[:, F:])
            elif rest == "block_sparse_moe.output_linear.weight":
                put(b + "ffn_down_exps.weight", a)
            else:
                e = re.match(r"mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$", rest)
                assert e, f"unmapped tensor {k}"
                sd.setdefault(("stack", b, e.group(2)), {})[int(e.group(1))] = a
    for key in [k for k in sd if isinstance(k, tuple)]:
        _, b, role = key
        put(b + f"ffn_{role}_exps.weight", np.stack([sd[key][i] for i in sorted(sd[key])]))
    gguf.write_gguf(path, meta, tensors)


FAMILY_CASES = ["olmo2", "olmoe", "smollm3", "granite", "granitemoe", "gemma2", "gemma3", "gpt_oss"]


def _put_all(path, meta, rows):
    gguf.write_gguf(path, meta, [_f32(n, a) for n, a in rows])


def _mpt_to_gguf(path, m):
    c = m.config
    meta = {"general.architecture": "mpt", "mpt.block_count": c.n_layers, "mpt.embedding_length": c.d_model, "mpt.attention.head_count": c.n_heads,
            "mpt.feed_forward_length": 4 * c.d_model, "mpt.attention.layer_norm_epsilon": float(c.layer_norm_epsilon),
            "mpt.attention.max_alibi_bias": float(c.attn_config.alibi_bias_max), "mpt.context_length": c.max_seq_len, "mpt.vocab_size": c.vocab_size}
    table = {"norm_1.weight": "attn_norm.weight", "norm_2.weight": "ffn_norm.weight", "attn.Wqkv.weight": "attn_qkv.weight",
             "attn.out_proj.weight": "attn_output.weight", "ffn.up_proj.weight": "ffn_up.weight", "ffn.down_proj.weight": "ffn_down.weight"}
    rows = []
    for k, v in m.state_dict().items():
        a = v.detach().float().numpy()
        mm = re.match(r"transformer\.blocks\.(\d+)\.(.+)$", k)
        if k == "transformer.wte.weight":
            rows.append(("token_embd.weight", a))
        elif k == "transformer.norm_f.weight":
            rows.append(("output_norm.weight", a))
        elif mm:
            rows.append((f"blk.{mm.group(1)}.{table[mm.group(2)]}", a))
    _put_all(path, meta, rows)


def _bloom_to_gguf(path, m):
    c = m.config
    nh, H = c.n_head, c.hidden_size
    meta = {"general.architecture": "bloom", "bloom.block_count": c.n_layer, "bloom.embedding_length": H, "bloom.attention.head_count": nh,
            "bloom.feed_forward_length": 4 * H, "bloom.attention.layer_norm_epsilon": float(c.layer_norm_epsilon), "bloom.vocab_size": c.vocab_size}
    table = {"input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm", "self_attention.dense": "attn_output",
             "mlp.dense_h_to_4h": "ffn_up", "mlp.dense_4h_to_h": "ffn_down", "self_attention.query_key_value": "attn_qkv"}
    top = {"transformer.word_embeddings.weight": "token_embd.weight", "transformer.word_embeddings_layernorm.weight": "token_embd_norm.weight",
           "transformer.word_embeddings_layernorm.bias": "token_embd_norm.bias", "transformer.ln_f.weight": "output_norm.weight",
           "transformer.ln_f.bias": "output_norm.bias"}
    rows = []
    for k, v in m.state_dict().items():
        a = v.detach().float().numpy()
        mm = re.match(r"transformer\.h\.(\d+)\.(.+)\.(weight|bias)$", k)
        if k in top:
            rows.append((top[k], a))
        elif mm:
            if mm.group(2) == "self_attention.query_key_value":      # the converter regroups [head][q | k | v] rows into thirds
                a = a.reshape(nh, 3, H // nh, -1) if a.ndim == 2 else a.reshape(nh, 3, H // nh)
                a = np.concatenate([a[:, i].reshape((H, -1) if a.ndim == 4 else (H,)) for i in range(3)], 0)
            rows.append((f"blk.{mm.group(1)}.{table[mm.group(2)]}.{mm.group(3)}", a))
    _put_all(path, meta, rows)


def _minimax_to_gguf(path, m):
    c = m.config
    arch = "minimax-m2"
    meta = {"general.architecture": arch, f"{arch}.block_count": c.num_hidden_layers, f"{arch}.embedding_length": c.hidden_size,
            f"{arch}.attention.head_count": c.num_attention_heads, f"{arch}.attention.head_count_kv": c.num_key_value_heads,
            f"{arch}.attention.key_length": c.head_dim, f"{arch}.feed_forward_length": c.intermediate_size,
            f"{arch}.expert_feed_forward_length": c.intermediate_size, f"{arch}.expert_count": c.num_local_experts,
            f"{arch}.expert_used_count": c.num_experts_per_tok, f"{arch}.expert_gating_func": 2,
            f"{arch}.rope.dimension_count": int(getattr(c, "rotary_dim", None) or c.head_dim),
            f"{arch}.rope.freq_base": float(c.rope_parameters["rope_theta"]), f"{arch}.attention.layer_norm_rms_epsilon": float(c.rms_norm_eps),
            f"{arch}.context_length": c.max_position_embeddings, f"{arch}.vocab_size": c.vocab_size}
    table = {**LAYER, "block_sparse_moe.gate.weight": "ffn_gate_inp.weight", "block_sparse_moe.e_score_correction_bias": "exp_probs_b.bias",
             "mlp.gate.weight": "ffn_gate_inp.weight", "mlp.e_score_correction_bias": "exp_probs_b.bias"}
    rows, stacks = [], {}
    for k, v in m.state_dict().items():
        a = v.detach().float().numpy()
        mm = re.match(r"model\.layers\.(\d+)\.(.+)$", k)
        if k == "model.embed_tokens.weight":
            rows.append(("token_embd.weight", a))
        elif k == "model.norm.weight":
            rows.append(("output_norm.weight", a))
        elif k == "lm_head.weight":
            rows.append(("output.weight", a))
        elif mm and mm.group(2) in table:
            rows.append((f"blk.{mm.group(1)}.{table[mm.group(2)]}", a))
        elif mm:
            e = re.match(r"(?:block_sparse_moe|mlp)\.experts\.(\d+)\.(w1|w2|w3|gate_proj|up_proj|down_proj)\.weight$", mm.group(2))
            if e:
                role = {"w1": "gate", "w3": "up", "w2": "down", "gate_proj": "gate", "up_proj": "up", "down_proj": "down"}[e.group(2)]
                stacks.setdefault((mm.group(1), role), {})[int(e.group(1))] = a
            elif mm.group(2).endswith("experts.gate_up_proj"):
                F = a.shape[1] // 2
                rows += [(f"blk.{mm.group(1)}.ffn_gate_exps.weight", a[:, :F]), (f"blk.{mm.group(1)}.ffn_up_exps.weight", a[:, F:])]
            elif mm.group(2).endswith("experts.down_proj"):
                rows.append((f"blk.{mm.group(1)}.ffn_down_exps.weight", a))
            else:
                raise AssertionError(f"unmapped tensor {k}")
    for (l, role), parts in stacks.items():
        rows.append((f"blk.{l}.ffn_{role}_exps.weight", np.stack([parts[i] for i in sorted(parts)])))
    _put_all(path, meta, rows)


def _deepseek2_to_gguf(path, m, split_kv_b):
    c = m.config
    arch = "deepseek2"
    nh, dn, dr, dv, r = c.num_attention_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank
    meta = {"general.architecture": arch, f"{arch}.block_count": c.num_hidden_layers, f"{arch}.embedding_length": c.hidden_size,
            f"{arch}.attention.head_count": nh, f"{arch}.attention.head_count_kv": 1 if split_kv_b else nh,
            f"{arch}.feed_forward_length": c.intermediate_size, f"{arch}.expert_feed_forward_length": c.moe_intermediate_size,
            f"{arch}.expert_count": c.n_routed_experts, f"{arch}.expert_used_count": c.num_experts_per_tok,
            f"{arch}.expert_shared_count": c.n_shared_experts, f"{arch}.leading_dense_block_count": c.first_k_dense_replace,
            f"{arch}.expert_weights_scale": float(c.routed_scaling_factor), f"{arch}.expert_weights_norm": bool(c.norm_topk_prob),
            f"{arch}.expert_gating_func": 1, f"{arch}.attention.kv_lora_rank": r, f"{arch}.rope.dimension_count": dr,
            f"{arch}.rope.freq_base": float(c.rope_parameters["rope_theta"]), f"{arch}.attention.layer_norm_rms_epsilon": float(c.rms_norm_eps),
            f"{arch}.context_length": c.max_position_embeddings, f"{arch}.vocab_size": c.vocab_size}
    if split_kv_b:      # the absorbed form: the plain keys describe the one latent head, the ``_mla`` keys the per-head widths
        meta.update({f"{arch}.attention.key_length": r + dr, f"{arch}.attention.value_length": r,
                     f"{arch}.attention.key_length_mla": dn + dr, f"{arch}.attention.value_length_mla": dv})
    else:
        meta.update({f"{arch}.attention.key_length": dn + dr, f"{arch}.attention.value_length": dv})
    if c.q_lora_rank:
        meta[f"{arch}.attention.q_lora_rank"] = c.q_lora_rank
    table = {"input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
             "self_attn.q_proj.weight": "attn_q.weight", "self_attn.q_a_proj.weight": "attn_q_a.weight",
             "self_attn.q_a_layernorm.weight": "attn_q_a_norm.weight", "self_attn.q_b_proj.weight": "attn_q_b.weight",
             "self_attn.kv_a_proj_with_mqa.weight": "attn_kv_a_mqa.weight", "self_attn.kv_a_layernorm.weight": "attn_kv_a_norm.weight",
             "self_attn.o_proj.weight": "attn_output.weight", "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
             "mlp.down_proj.weight": "ffn_down.weight", "mlp.gate.weight": "ffn_gate_inp.weight",
             "mlp.shared_experts.gate_proj.weight": "ffn_gate_shexp.weight", "mlp.shared_experts.up_proj.weight": "ffn_up_shexp.weight",
             "mlp.shared_experts.down_proj.weight": "ffn_down_shexp.weight"}
    rows, stacks = [], {}
    for k, v in m.state_dict().items():
        a = v.detach().float().numpy()
        mm = re.match(r"model\.layers\.(\d+)\.(.+)$", k)
        if k == "model.embed_tokens.weight":
            rows.append(("token_embd.weight", a))
        elif k == "model.norm.weight":
            rows.append(("output_norm.weight", a))
        elif k == "lm_head.weight":
            rows.append(("output.weight", a))
        elif mm and mm.group(2) in table:
            rows.append((f"blk.{mm.group(1)}.{table[mm.group(2)]}", a))
        elif mm and mm.group(2) == "self_attn.kv_b_proj.weight":
            if split_kv_b:
                kv = a.reshape(nh, dn + dv, r)
                rows += [(f"blk.{mm.group(1)}.attn_k_b.weight", np.ascontiguousarray(kv[:, :dn].transpose(0, 2, 1))),
                         (f"blk.{mm.group(1)}.attn_v_b.weight", np.ascontiguousarray(kv[:, dn:]))]
            else:
                rows.append((f"blk.{mm.group(1)}.attn_kv_b.weight", a))
        elif mm:
            e = re.match(r"mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$", mm.group(2))
            if e:
                stacks.setdefault((mm.group(1), e.group(2)), {})[int(e.group(1))] = a
            elif mm.group(2) == "mlp.experts.gate_up_proj":
                F = a.shape[1] // 2
                rows += [(f"blk.{mm.group(1)}.ffn_gate_exps.weight", a[:, :F]), (f"blk.{mm.group(1)}.ffn_up_exps.weight", a[:, F:])]
            elif mm.group(2) == "mlp.experts.down_proj":
                rows.append((f"blk.{mm.group(1)}.ffn_down_exps.weight", a))
            else:
                raise AssertionError(f"unmapped tensor {k}")
    for (l, role), parts in stacks.items():
        rows.append((f"blk.{l}.ffn_{role}_exps.weight", np.stack([parts[i] for i in sorted(parts)])))
    _put_all(path, meta, rows)


def _qwen35_to_gguf(path, m, nextn):
    """llama.cpp's ``qwen35`` layout: the delta-net quantities one tensor each with the value heads tiled over the key
    heads, ``ssm_a = -exp(A_log)``, every ``1 + w`` norm with the one folded in, and (``nextn``) one more block after the stack."""
    c = m.config
    arch = "qwen35"
    nk, nv, Dg, K = c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim, c.linear_conv_kernel_dim
    H, L, rep, kd = c.hidden_size, c.num_hidden_layers, nv // nk, nk * Dg
    tiled = [(t % nk) * rep + t // nk for t in range(nv)]                 # the grouped head each tiled position holds

    def tile(a, block):
        return a.reshape(nv, block, -1)[tiled].reshape(a.shape)

    rp = c.rope_parameters
    meta = {"general.architecture": arch, f"{arch}.block_count": L + (1 if nextn else 0), f"{arch}.embedding_length": H,
            f"{arch}.attention.head_count": c.num_attention_heads, f"{arch}.attention.head_count_kv": c.num_key_value_heads,
            f"{arch}.attention.key_length": c.head_dim, f"{arch}.feed_forward_length": c.intermediate_size,
            f"{arch}.rope.freq_base": float(rp["rope_theta"]), f"{arch}.rope.dimension_count": int(c.head_dim * rp.get("partial_rotary_factor", 1.0)),
            f"{arch}.attention.layer_norm_rms_epsilon": float(c.rms_norm_eps), f"{arch}.context_length": c.max_position_embeddings,
            f"{arch}.vocab_size": c.vocab_size, f"{arch}.ssm.inner_size": nv * Dg, f"{arch}.ssm.state_size": Dg, f"{arch}.ssm.group_count": nk,
            f"{arch}.ssm.time_step_rank": nv, f"{arch}.ssm.conv_kernel": K, f"{arch}.full_attention_interval": 2}
    if nextn:
        meta[f"{arch}.nextn_predict_layers"] = 1
    sd = {k: v.detach().float().numpy() for k, v in m.state_dict().items()}
    rows = [("token_embd.weight", sd["model.embed_tokens.weight"]), ("output_norm.weight", sd["model.norm.weight"] + 1.0),
            ("output.weight", sd["lm_head.weight"])]
    for l in range(L):
        hf, b = f"model.layers.{l}.", f"blk.{l}."
        rows += [(b + "attn_norm.weight", sd[hf + "input_layernorm.weight"] + 1.0),
                 (b + "post_attention_norm.weight", sd[hf + "post_attention_layernorm.weight"] + 1.0)]
        if hf + "self_attn.q_proj.weight" in sd:
            for gg, name in (("attn_q", "q_proj"), ("attn_k", "k_proj"), ("attn_v", "v_proj"), ("attn_output", "o_proj")):
                rows.append((b + gg + ".weight", sd[hf + f"self_attn.{name}.weight"]))
            rows += [(b + "attn_q_norm.weight", sd[hf + "self_attn.q_norm.weight"] + 1.0), (b + "attn_k_norm.weight", sd[hf + "self_attn.k_norm.weight"] + 1.0)]
        else:
            la = hf + "linear_attn."
            qkv = sd[la + "in_proj_qkv.weight"]
            conv = sd[la + "conv1d.weight"].reshape(2 * kd + nv * Dg, K)
            rows += [(b + "attn_qkv.weight", np.concatenate([qkv[:2 * kd], tile(qkv[2 * kd:], Dg)], 0)),
                     (b + "attn_gate.weight", tile(sd[la + "in_proj_z.weight"], Dg)), (b + "ssm_beta.weight", tile(sd[la + "in_proj_b.weight"], 1)),
                     (b + "ssm_alpha.weight", tile(sd[la + "in_proj_a.weight"], 1)), (b + "ssm_dt.bias", tile(sd[la + "dt_bias"], 1)),
                     (b + "ssm_a", tile(-np.exp(sd[la + "A_log"]), 1)),
                     (b + "ssm_conv1d.weight", np.concatenate([conv[:2 * kd], tile(conv[2 * kd:], Dg)], 0)),
                     (b + "ssm_norm.weight", sd[la + "norm.weight"]),
                     (b + "ssm_out.weight", np.ascontiguousarray(tile(np.ascontiguousarray(sd[la + "out_proj.weight"].T), Dg).T))]
        for gg, name in (("ffn_gate", "gate_proj"), ("ffn_up", "up_proj"), ("ffn_down", "down_proj")):
            rows.append((b + gg + ".weight", sd[hf + f"mlp.{name}.weight"]))
    if nextn:                                                              # never read: it is not part of the stack
        rows += [(f"blk.{L}.attn_norm.weight", np.ones(H, np.float32)), (f"blk.{L}.nextn.eh_proj.weight", np.ones((H, 2 * H), np.float32)),
                 (f"blk.{L}.attn_qkv.weight", np.ones((3, H), np.float32))]
    _put_all(path, meta, rows)


GEMMA4_LAYER = {"input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "post_attention_norm.weight",
                "pre_feedforward_layernorm.weight": "ffn_norm.weight", "post_feedforward_layernorm.weight": "post_ffw_norm.weight",
                "layer_scalar": "layer_output_scale.weight", "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
                "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight", "self_attn.q_norm.weight": "attn_q_norm.weight",
                "self_attn.k_norm.weight": "attn_k_norm.weight", "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
                "mlp.down_proj.weight": "ffn_down.weight", "pre_feedforward_layernorm_2.weight": "ffn_pre_norm_2.weight",
                "post_feedforward_layernorm_1.weight": "ffn_post_norm_1.weight", "post_feedforward_layernorm_2.weight": "ffn_post_norm_2.weight",
                "router.proj.weight": "ffn_gate_inp.weight", "router.scale": "ffn_gate_inp.scale", "router.per_expert_scale": "ffn_down_exps.scale",
                "experts.gate_up_proj": "ffn_gate_up_exps.weight", "experts.down_proj": "ffn_down_exps.weight"}


def _gemma4_to_gguf(path, m):
    """llama.cpp's ``gemma4`` layout: per-layer K/V head counts and sliding flags as arrays, the two head widths, no ``attn_v``
    on a global layer that reads its value from the key projection, and the global layers' rotary tail as ``rope_freqs.weight``
    (ones over the rotated pairs, 1e30 over the rest)."""
    c = m.config
    arch = "gemma4"
    local = [t == "sliding_attention" for t in c.layer_types]
    rp = c.rope_parameters
    meta = {"general.architecture": arch, f"{arch}.block_count": c.num_hidden_layers, f"{arch}.embedding_length": c.hidden_size,
            f"{arch}.feed_forward_length": c.intermediate_size, f"{arch}.context_length": c.max_position_embeddings,
            f"{arch}.attention.head_count": c.num_attention_heads,
            f"{arch}.attention.head_count_kv": [int(c.num_key_value_heads if loc else (c.num_global_key_value_heads or c.num_key_value_heads)) for loc in local],
            f"{arch}.attention.sliding_window_pattern": local, f"{arch}.attention.sliding_window": c.sliding_window,
            f"{arch}.attention.key_length": c.global_head_dim, f"{arch}.attention.key_length_swa": c.head_dim,
            f"{arch}.rope.freq_base": float(rp["full_attention"]["rope_theta"]), f"{arch}.rope.freq_base_swa": float(rp["sliding_attention"]["rope_theta"]),
            f"{arch}.attention.layer_norm_rms_epsilon": float(c.rms_norm_eps), f"{arch}.vocab_size": c.vocab_size}
    if c.final_logit_softcapping:
        meta[f"{arch}.final_logit_softcapping"] = float(c.final_logit_softcapping)
    if c.enable_moe_block:
        meta.update({f"{arch}.expert_count": c.num_experts, f"{arch}.expert_used_count": c.top_k_experts,
                     f"{arch}.expert_feed_forward_length": c.moe_intermediate_size})
    pairs = c.global_head_dim // 2
    rotated = int(pairs * rp["full_attention"].get("partial_rotary_factor", 1.0))
    rows = [("rope_freqs.weight", np.array([1.0] * rotated + [1e30] * (pairs - rotated), np.float32))]
    for k, v in m.state_dict().items():
        a = v.detach().float().numpy()
        mm = re.match(r"model\.layers\.(\d+)\.(.+)$", k)
        if k == "model.embed_tokens.weight":
            rows.append(("token_embd.weight", a))
        elif k == "model.norm.weight":
            rows.append(("output_norm.weight", a))
        elif mm:
            l = int(mm.group(1))
            if mm.group(2) == "self_attn.v_proj.weight" and c.attention_k_eq_v and not local[l]:
                continue
            rows.append((f"blk.{l}.{GEMMA4_LAYER[mm.group(2)]}", a))
    _put_all(path, meta, rows)


@pytest.mark.parametrize("case", ["gemma4-value-is-key", "gemma4-moe"])
def test_gemma4_gguf_equals_the_hugging_face_forward(case, tmp_path):
    m, vocab = build(CASES[case])
    toks = torch.randint(0, vocab, (1, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(toks).logits[0].numpy()
    path = str(tmp_path / "gemma4.gguf")
    _gemma4_to_gguf(path, m)
    h = ModelHandle.load(path)
    assert h.cfg.family == "gemma4" and h.cfg.k_eq_v == bool(m.config.attention_k_eq_v) and h.cfg.tie_embeddings
    sess = OracleSession(h.model, h.oracle_weights(), capacity=32)
    sess._graph = lambda T, embeds=False: h.model.trace(StepSpec(rows=1, tokens=T, capacity=32, logit_rows="all"))
    got = sess.step(toks.numpy()).reshape(ref.shape)
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err < 2e-5, err


@pytest.mark.parametrize("nextn", [False, True])
def test_qwen35_gguf_equals_the_hugging_face_forward(nextn, tmp_path):
    m, vocab = build(CASES["qwen3_5"])
    toks = torch.randint(0, vocab, (1, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(toks).logits[0].numpy()
    path = str(tmp_path / "qwen35.gguf")
    _qwen35_to_gguf(path, m, nextn)
    h = ModelHandle.load(path)
    assert h.cfg.family == "qwen38_27b" and h.cfg.n_layers == m.config.num_hidden_layers and h.cfg.norm_offset == 0.0
    assert not any(k.startswith(f"layers.{h.cfg.n_layers}.") for k in h.canonical)
    sess = OracleSession(h.model, h.oracle_weights(), capacity=32)
    sess._graph = lambda T, embeds=False: h.model.trace(StepSpec(rows=1, tokens=T, capacity=32, logit_rows="all"))
    got = sess.step(toks.numpy()).reshape(ref.shape)
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err < 1e-4, err


@pytest.mark.parametrize("family", ["mpt", "bloom", "minimax_m2", "deepseek2", "deepseek2-absorbed"])
def test_gguf_of_the_families_with_their_own_layouts(family, tmp_path):
    """MPT and BLOOM (LayerNorm stacks with a fused ``attn_qkv``, BLOOM's regrouped into thirds by the converter and with
    biases everywhere), MiniMax-M2 (sigmoid router with ``exp_probs_b``, partial rotary) and DeepSeek-V2 (latent attention
    rows; the up-projection stored whole or, in the absorbed form, as ``attn_k_b`` / ``attn_v_b`` per head)."""
    name = family.split("-")[0]
    m, vocab = build(CASES[name])
    toks = torch.randint(0, vocab, (1, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(toks).logits[0].numpy()
    path = str(tmp_path / f"{family}.gguf")
    if name == "mpt":
        _mpt_to_gguf(path, m)
    elif name == "bloom":
        _bloom_to_gguf(path, m)
    elif name == "minimax_m2":
        _minimax_to_gguf(path, m)
    else:
        _deepseek2_to_gguf(path, m, split_kv_b=family.endswith("absorbed"))
    h = ModelHandle.load(path)
    assert h.cfg.family == name and h.kind == "gguf"
    sess = OracleSession(h.model, h.oracle_weights(), capacity=32)
    sess._graph = lambda T, embeds=False: h.model.trace(StepSpec(rows=1, tokens=T, capacity=32, logit_rows="all"))
    got = sess.step(toks.numpy()).reshape(ref.shape)
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err < 2e-5, err


@pytest.mark.parametrize("family", FAMILY_CASES)
def test_gguf_of_the_family_equals_the_hugging_face_forward(family, tmp_path):
    case = dict(CASES["smollm3-nope-layer" if family == "smollm3" else family])
    if family == "gemma2":
        case["query_pre_attn_scalar"] = BASE["head_dim"]          # a GGUF carries no query scalar: it is the head width
    if family == "gemma3":
        case["query_pre_attn_scalar"] = BASE["head_dim"]
        case["num_hidden_layers"], case["layer_types"] = 6, ["sliding_attention"] * 5 + ["full_attention"]   # the pattern a GGUF implies
    if family == "gpt_oss":
        case["sliding_window"] = 6
    if family == "smollm3":
        case["num_hidden_layers"], case["no_rope_layers"], case["no_rope_layer_interval"] = 4, [1, 1, 1, 0], 4
    m, vocab = build(case)
    toks = torch.randint(0, vocab, (1, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(toks).logits[0].numpy()
    path = str(tmp_path / f"{family}.gguf")
    _to_gguf(path, family, m)
    h = ModelHandle.load(path)
    assert h.cfg.family == ("granite" if family == "granitemoe" else family) and h.kind == "gguf"
    sess = OracleSession(h.model, h.oracle_weights(), capacity=32)
    sess._graph = lambda T, embeds=False: h.model.trace(StepSpec(rows=1, tokens=T, capacity=32, logit_rows="all"))
    got = sess.step(toks.numpy()).reshape(ref.shape)
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err < 2e-5, err


def test_quantised_gguf_of_a_new_family_generates_packed(tmp_path):
    """A Q8_0 OLMoE GGUF through the packed oracle: the projections stay as stored and generation equals the oracle over
    the decoded weights."""
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.llm import LLM
    m, vocab = build({**CASES["olmoe"], "hidden_size": 128, "head_dim": 32, "intermediate_size": 64})
    path = str(tmp_path / "olmoe-q8.gguf")
    _to_gguf(path, "olmoe", m, quantise="Q8_0")
    prompt = [int(t) for t in np.random.default_rng(0).integers(3, vocab, 18)]
    p = SamplingParams(max_tokens=5, ignore_eos=True)
    want = LLM.oracle(path, rows=1, max_seq=64, num_blocks=8, prefill_chunk=16).generate_tokens(prompt, p)
    assert LLM.oracle(path, rows=1, max_seq=64, num_blocks=8, prefill_chunk=16, packed=True).generate_tokens(prompt, p) == want
