"""The supported-models page, generated from the registry (``python -m poot_b200.models.support_matrix`` prints it;
``docs/supported-models.md`` is the committed copy and a test keeps it current).  The reference generates its page
the same way (website/docs/develop/supported-models.md:32-79)."""
from __future__ import annotations

from .registry import GGUF_FAMILIES, Registry

# header fields of a representative checkpoint of each family, enough to build its configuration
SAMPLES = {
    "llama": dict(model_type="llama"), "qwen2": dict(model_type="qwen2"), "qwen3": dict(model_type="qwen3"),
    "olmo2": dict(model_type="olmo2"), "phi3": dict(model_type="phi3"), "smollm3": dict(model_type="smollm3", no_rope_layers=[1, 1, 1, 0]),
    "granite": dict(model_type="granite", attention_multiplier=0.0078125),
    "mpt": dict(model_type="mpt", d_model=4096, n_heads=32, n_layers=4, attn_config={"alibi": True}),
    "bloom": dict(model_type="bloom", n_head=32, n_layer=4),
    "gemma2": dict(model_type="gemma2", query_pre_attn_scalar=128, sliding_window=4096, attn_logit_softcapping=50.0, final_logit_softcapping=30.0),
    "gemma3": dict(model_type="gemma3_text", query_pre_attn_scalar=128, sliding_window=1024),
    "qwen3moe": dict(model_type="qwen3_moe", num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768),
    "gpt_oss": dict(model_type="gpt_oss", num_local_experts=32, num_experts_per_tok=4, sliding_window=128, attention_bias=True),
    "olmoe": dict(model_type="olmoe", num_experts=64, num_experts_per_tok=8),
    "minimax_m2": dict(model_type="minimax_m2", num_local_experts=256, num_experts_per_tok=8),
    "deepseek2": dict(model_type="deepseek_v2", n_routed_experts=64, num_experts_per_tok=6, moe_intermediate_size=1408, kv_lora_rank=512,
                      q_lora_rank=None, qk_rope_head_dim=64, qk_nope_head_dim=128, v_head_dim=128, n_shared_experts=2, first_k_dense_replace=1),
    "deepseek3": dict(model_type="deepseek_v3", n_routed_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048, kv_lora_rank=512,
                      q_lora_rank=1536, qk_rope_head_dim=64, qk_nope_head_dim=128, v_head_dim=128, n_shared_experts=1, n_group=8,
                      topk_group=4, first_k_dense_replace=3),
    "deepseek32": dict(model_type="deepseek_v32", n_routed_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048, kv_lora_rank=512,
                       q_lora_rank=1536, qk_rope_head_dim=64, qk_nope_head_dim=128, v_head_dim=128, n_shared_experts=1, n_group=8,
                       topk_group=4, first_k_dense_replace=3, index_topk=2048, index_n_heads=64, index_head_dim=128),
    "glm_moe_dsa": dict(model_type="glm_moe_dsa", n_routed_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048,
                        kv_lora_rank=512, q_lora_rank=2048, qk_rope_head_dim=64, qk_nope_head_dim=192, v_head_dim=256,
                        n_shared_experts=1, mlp_layer_types=["dense", "sparse", "sparse", "sparse"], index_topk=2048,
                        index_n_heads=32, index_head_dim=128),
    "nemotron_h": dict(model_type="nemotron_h", hybrid_override_pattern="M-M*", mamba_num_heads=128, mamba_head_dim=64, ssm_state_size=128, n_groups=8),
    "qwen3next": dict(model_type="qwen3_next", linear_num_value_heads=32, linear_num_key_heads=16, linear_key_head_dim=128,
                      linear_value_head_dim=128, num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
                      shared_expert_intermediate_size=512),
    "qwen38_27b": dict(model_type="qwen3_5_text", linear_num_value_heads=48, linear_num_key_heads=16, linear_key_head_dim=128,
                       linear_value_head_dim=128),
    "qwen_vl": dict(model_type="qwen2_5_vl", text_config=dict(hidden_size=2048, num_hidden_layers=4, num_attention_heads=16,
                                                              num_key_value_heads=2, intermediate_size=11008, vocab_size=151936,
                                                              rope_parameters={"rope_type": "default", "mrope_section": [16, 24, 24],
                                                                               "rope_theta": 1000000.0}),
                    vision_config=dict(depth=32, hidden_size=1280, intermediate_size=3420, num_heads=16, out_hidden_size=2048),
                    image_token_id=151655),
    "gemma4": dict(model_type="gemma4_text", head_dim=256, global_head_dim=512, hidden_size_per_layer_input=256, num_kv_shared_layers=2,
                   vocab_size_per_layer_input=32000, sliding_window=512,
                   layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    "glm53_flash": dict(model_type="glm5_next", text_config=dict(
        vocab_size=151552, hidden_size=2048, num_hidden_layers=4, num_nextn_predict_layers=1, max_position_embeddings=131072,
        layer_types=["linear_attention", "linear_attention", "linear_attention", "deepseek_sparse_attention"],
        mlp_layer_types=["dense", "sparse", "sparse", "sparse"],
        linear_attn_config=dict(num_heads=32, head_dim=128, short_conv_kernel_size=4, gate_lower_bound=-5.0), hc_mult=4,
        hc_sinkhorn_iters=20, num_attention_heads=32, q_lora_rank=1024, kv_lora_rank=512, qk_nope_head_dim=192, qk_rope_head_dim=0,
        v_head_dim=128, index_n_heads=32, index_head_dim=128, index_topk=2048, index_kpool=4, intermediate_size=10240,
        moe_intermediate_size=1536, n_routed_experts=128, num_experts_per_tok=8, n_shared_experts=1, routed_scaling_factor=2.5)),
    "deepseek4": dict(model_type="deepseek_v4", vocab_size=129280, hidden_size=4096, num_hidden_layers=4, num_attention_heads=64,
                      head_dim=512, qk_rope_head_dim=64, q_lora_rank=1024, o_groups=8, o_lora_rank=1024, sliding_window=128,
                      compress_ratios=[0, 4, 128, 4], index_n_heads=64, index_head_dim=128, index_topk=512, hc_mult=4,
                      hc_sinkhorn_iters=20, n_routed_experts=256, num_experts_per_tok=6, moe_intermediate_size=2048,
                      n_shared_experts=1, routed_scaling_factor=1.5, num_hash_layers=1, max_position_embeddings=1048576),
    "qwen38": dict(model_type="qwen4_exp", text_config=dict(
        vocab_size=151936, hidden_size=2048, num_hidden_layers=4, num_attention_heads=16, num_key_value_heads=2, head_dim=256,
        partial_rotary_factor=0.25, max_position_embeddings=262144,
        layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"], linear_num_key_heads=16,
        linear_num_value_heads=32, linear_key_head_dim=128, linear_value_head_dim=128, output_gate_type="sigmoid", num_experts=256,
        num_experts_per_tok=8, moe_intermediate_size=512, shared_expert_intermediate_size=512, hc_count=4, hc_lowrank=32,
        indexer_n_heads=16, indexer_head_dim=128, indexer_budget=2048, indexer_compress_ratio=64, ple_layer_ids=[1, 3],
        ple_embed_dim=1024, ple_conv_kernel_size=4, ngram_size=3, heads_per_ngram=8, ngram_vocab_size_base=500000,
        make_ngram_vocab_size_divisible_by=128, eos_token_id=151645)),
    "bert": dict(model_type="bert", num_attention_heads=12, intermediate_size=3072, hidden_size=768),
    "idefics3": dict(model_type="idefics3", text_config=dict(model_type="llama", hidden_size=2048, num_hidden_layers=4,
                                                             num_attention_heads=32, num_key_value_heads=32, intermediate_size=8192,
                                                             vocab_size=49155),
                     vision_config=dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=27, num_attention_heads=16,
                                        image_size=384, patch_size=14), scale_factor=3, image_token_id=49153),
}
# Families whose device program has run on a B200 against the fp32 restatement (the GPU tests that are plain tests, not
# expected-failure marks).  Every other family with a device program has so far only run on the host-emulated kernels.
DEVICE_VERIFIED = {"llama", "qwen3"}


def device_state(name: str, has_program: bool) -> str:
    if not has_program:
        return "general executor only"
    return "device-verified" if name in DEVICE_VERIFIED else "emulated only"


BASE = dict(hidden_size=4096, num_hidden_layers=4, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
            intermediate_size=14336, vocab_size=32000, max_position_embeddings=8192)


def rows():
    reg = Registry.builtin()
    out = []
    for e in reg.entries:
        if e.from_hf is None:
            out.append((e.name, ", ".join(e.hf_types), "refused", "-", "-", f"needs {e.missing}"))
            continue
        sample = SAMPLES[e.name]
        header = sample if e.name in ("mpt", "bloom") else {**BASE, **sample}
        if e.name in ("mpt", "bloom"):
            header = {"vocab_size": 32000, "hidden_size": 4096, **header}
        model = reg.resolve_hf(header)
        if e.kind == "encoder":
            out.append((e.name, ", ".join(e.hf_types), "oracle + device", "no", device_state(e.name, True), "- (embeddings and rerank scores; head widths that are multiples of 32)"))
            continue
        if e.kind == "vlm" and model.cfg.mrope_sections:
            out.append((e.name, ", ".join(e.hf_types), "oracle + device", "no", "text stack, " + device_state(e.name, True),
                        "a device program for the vision tower (it is evaluated on the host, once per image)"))
            continue
        if e.kind == "vlm":
            out.append((e.name, ", ".join(e.hf_types), "oracle + device", "no", device_state(e.name, True),
                        "vision towers whose heads are not multiples of 32 wide run on the host evaluator"))
            continue
        gaps = model.cfg.device_gaps()
        device = device_state(e.name, not gaps)
        out.append((e.name, ", ".join(e.hf_types), "oracle + device" if not gaps else "oracle", "yes" if e.name in GGUF_FAMILIES else "no",
                    device, "; ".join(gaps) if gaps else "-"))
    return out


def render() -> str:
    lines = ["# Supported model families", "",
             "Generated by `python -m poot_b200.models.support_matrix`; do not edit by hand.", "",
             "`oracle`: traced into the graph IR and evaluated by the CPU oracle (`--backend oracle`), checked against the",
             "Hugging Face implementation.  `device`: the B200 engine has a kernel program for the family.  The `B200 engine`",
             "column says how far that program has been checked: `device-verified` = it ran on a B200 and matched the fp32",
             "restatement; `emulated only` = the engine's unmodified program ran on host restatements of the kernels and",
             "matched the oracle and Hugging Face, but has not run on a device yet; `general executor only` = no hand-written",
             "program: the family runs on the device through the general executor (`--backend graph`, one launch per equation).  The last",
             "column names what the device program lacks for a representative checkpoint of the family.", "",
             "| family | header `model_type` | runs on | GGUF | B200 engine | missing on the device |", "|---|---|---|---|---|---|"]
    for r in rows():
        lines.append("| " + " | ".join(r) + " |")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    print(render(), end="")
