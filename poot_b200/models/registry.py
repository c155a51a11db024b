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
    kind: str = "decoder"             # decoder (standard stack) | encoder (embeddings / rerank scores) | vlm (vision tower + decoder) | own (a tracer of its own)
    tracer: Optional[str] = None      # kind "own": ``module:Class`` under ``models`` whose instances trace the family


def _rope_params(c: dict, layer_type: Optional[str] = None) -> dict:
    """Rotary settings of a header in either spelling: top-level ``rope_theta`` + ``rope_scaling`` (older
    checkpoints) or one ``rope_parameters`` table, optionally keyed by layer type (gemma3)."""
    rp = c.get("rope_parameters")
    if isinstance(rp, dict):
        if layer_type is not None and isinstance(rp.get(layer_type), dict):
            rp = rp[layer_type]
        elif rp and all(isinstance(v, dict) for v in rp.values()):
            rp = rp.get("full_attention") or next(iter(rp.values()))
        return dict(rp)
    out = dict(c.get("rope_scaling") or {})
    if "rope_theta" in c:
        out["rope_theta"] = c["rope_theta"]
    if "partial_rotary_factor" in c:
        out["partial_rotary_factor"] = c["partial_rotary_factor"]
    return out


def _rope_scaling(c: dict, rs: Optional[dict] = None) -> RopeScaling:
    rs = _rope_params(c) if rs is None else rs
    kind = rs.get("rope_type", rs.get("type", "none")) or "none"
    if kind == "default":
        kind = "none"
    return RopeScaling(kind=kind, factor=float(rs.get("factor", 1.0)),
                       low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                       high_freq_factor=float(rs.get("high_freq_factor", 4.0)),
                       original_max_position=int(rs.get("original_max_position_embeddings") or
                                                 c.get("original_max_position_embeddings") or 8192),
                       beta_fast=float(rs.get("beta_fast") or 32.0), beta_slow=float(rs.get("beta_slow") or 1.0),
                       attention_factor=rs.get("attention_factor"), short_factor=rs.get("short_factor"),
                       long_factor=rs.get("long_factor"))


def _token(v, default: int) -> int:
    if isinstance(v, (list, tuple)):
        v = v[0] if v else None
    return default if v is None else int(v)


def _windows(c: dict, n_layers: int) -> Optional[list]:
    """Per-layer sliding windows from ``layer_types`` (``sliding_attention`` layers use ``sliding_window``)."""
    lt, win = c.get("layer_types"), int(c.get("sliding_window") or 0)
    if not lt or not win or not c.get("use_sliding_window", True):
        return None
    ws = [win if t in ("sliding_attention", "chunked_attention") else 0 for t in lt][:n_layers]
    return ws if len(set(ws)) > 1 else None


def _base(c: dict, family: str, **over) -> DecoderConfig:
    H, nh = c["hidden_size"], c["num_attention_heads"]
    rp = _rope_params(c)
    D = c.get("head_dim") or H // nh
    prf = float(rp.get("partial_rotary_factor") or 1.0)
    L = c["num_hidden_layers"]
    lw = _windows(c, L)
    win = int(c.get("sliding_window") or 0) if c.get("use_sliding_window", True) else 0
    if lw is None and c.get("layer_types") and all(t == "full_attention" for t in c["layer_types"]):
        win = 0
    cfg = DecoderConfig(
        name=c.get("_name_or_path", family) or family, family=family, n_layers=L, hidden=H,
        n_heads=nh, n_kv_heads=c.get("num_key_value_heads") or nh, head_dim=D,
        ffn=c.get("intermediate_size", 4 * H), vocab=c["vocab_size"], norm_eps=float(c.get("rms_norm_eps", 1e-6)),
        rope_theta=float(rp.get("rope_theta", 10000.0)), rope_scaling=_rope_scaling(c, rp),
        rope_dim=None if prf == 1.0 else int(D * prf),
        max_position=int(c.get("max_position_embeddings", 8192)), tie_embeddings=bool(c.get("tie_word_embeddings", False)),
        sliding_window=0 if lw is not None else win, layer_windows=lw,
        bos_token=_token(c.get("bos_token_id"), 1), eos_token=_token(c.get("eos_token_id"), 2))
    if c.get("attention_bias"):
        cfg.attn_bias = cfg.out_bias = True
    if c.get("mlp_bias"):
        cfg.mlp_bias = True
    for k, v in over.items():
        setattr(cfg, k, v)
    return cfg


def _experts(c: dict) -> int:
    return int(c.get("num_local_experts") or c.get("num_experts") or c.get("n_routed_experts") or 0)


def _llama(c: dict) -> DecoderConfig:
    cfg = _base(c, "llama")
    if _experts(c) > 0:   # Mixtral rides the llama entry (llama.rs:136-208)
        cfg.family, cfg.n_experts, cfg.top_k, cfg.moe_ffn = "mixtral", _experts(c), c["num_experts_per_tok"], c["intermediate_size"]
    return cfg


def _qwen2(c): return _base(c, "qwen2", attn_bias=True, out_bias=False)
def _qwen3(c): return _base(c, "qwen3", qk_norm=True, out_bias=False)
def _olmo2(c): return _base(c, "olmo2", qk_norm=True, qk_norm_wide=True, block="post")
def _phi3(c): return _base(c, "phi3")


def _smollm3(c):
    nr = c.get("no_rope_layers")
    return _base(c, "smollm3", rope_layers=[int(x) for x in nr] if nr and not all(nr) else None)


def _qwen3moe(c):
    return _base(c, "qwen3moe", qk_norm=True, out_bias=False, n_experts=_experts(c), top_k=c["num_experts_per_tok"],
                 moe_ffn=c["moe_intermediate_size"], norm_topk_prob=bool(c.get("norm_topk_prob", False)))


def _granite(c):
    cfg = _base(c, "granite", embed_scale=float(c.get("embedding_multiplier", 1.0)),
                residual_scale=float(c.get("residual_multiplier", 1.0)),
                logit_scale=1.0 / float(c.get("logits_scaling", 1.0)))
    if c.get("attention_multiplier") is not None:
        cfg.attn_scale = float(c["attention_multiplier"])
    if _experts(c) > 0:   # granitemoe: top-k logits, softmax over the selected ones
        cfg.n_experts, cfg.top_k, cfg.moe_ffn = _experts(c), c["num_experts_per_tok"], c["intermediate_size"]
    return cfg


def _olmoe(c):
    return _base(c, "olmoe", qk_norm=True, qk_norm_wide=True, n_experts=_experts(c), top_k=c["num_experts_per_tok"],
                 moe_ffn=c["intermediate_size"], norm_topk_prob=bool(c.get("norm_topk_prob", False)))


def _gemma(c, family: str) -> DecoderConfig:
    H = c["hidden_size"]
    lt = c.get("layer_types")
    L = c["num_hidden_layers"]
    if not lt:      # older headers: gemma2 alternates starting with a windowed layer; gemma3 has one global layer in six
        pat = int(c.get("sliding_window_pattern") or c.get("_sliding_window_pattern") or (2 if family == "gemma2" else 6))
        lt = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(L)]
    c = {**c, "layer_types": lt}
    cfg = _base(c, family, block="sandwich", act="gelu_tanh", embed_scale=float(H) ** 0.5, norm_offset=1.0,
                attn_scale=float(c.get("query_pre_attn_scalar") or (c.get("head_dim") or H // c["num_attention_heads"])) ** -0.5,
                attn_softcap=float(c.get("attn_logit_softcapping") or 0.0),
                final_softcap=float(c.get("final_logit_softcapping") or 0.0),
                tie_embeddings=bool(c.get("tie_word_embeddings", True)))
    if cfg.layer_windows is None and cfg.sliding_window == 0 and c.get("sliding_window") and all(t != "full_attention" for t in lt):
        cfg.sliding_window = int(c["sliding_window"])
    if family == "gemma3":
        cfg.qk_norm = True
        g = _rope_params(c, "full_attention")
        loc = _rope_params(c, "sliding_attention")
        cfg.rope_theta, cfg.rope_scaling = float(g.get("rope_theta", 1e6)), _rope_scaling(c, g)
        cfg.rope_theta_local = float(c.get("rope_local_base_freq") or loc.get("rope_theta", 10000.0))
    return cfg


def _gemma2(c): return _gemma(c, "gemma2")
def _gemma3(c): return _gemma(c, "gemma3")


def _gemma4(c):
    """Gemma 4 text stack (``gemma4_text``, or the text part of a multimodal ``gemma4`` header)."""
    from .gemma4 import Gemma4Config
    c = c.get("text_config") or c
    if c.get("use_bidirectional_attention") == "all":
        raise UnsupportedFamily("gemma4 with bidirectional attention over every token")
    L, H = c["num_hidden_layers"], c["hidden_size"]
    lt = list(c.get("layer_types") or ["full_attention"] * L)[:L]
    win = int(c.get("sliding_window") or 0)
    rp = c.get("rope_parameters") or {}
    full, local = dict(rp.get("full_attention") or {}), dict(rp.get("sliding_attention") or {})
    if full.get("rope_type", "default") not in ("default", "proportional") or local.get("rope_type", "default") != "default":
        raise UnsupportedFamily(f"gemma4 rope types {full.get('rope_type')!r} / {local.get('rope_type')!r}")
    act = {"gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_tanh", "gelu": "gelu_erf", "silu": "silu"}.get(
        c.get("hidden_activation", "gelu_pytorch_tanh"))
    if act is None:
        raise UnsupportedFamily(f"gemma4 activation {c.get('hidden_activation')!r}")
    moe = bool(c.get("enable_moe_block"))
    cap = c.get("final_logit_softcapping")
    return Gemma4Config(
        name="gemma4", family="gemma4", n_layers=L, hidden=H, n_heads=c["num_attention_heads"],
        n_kv_heads=c.get("num_key_value_heads") or c["num_attention_heads"], head_dim=c.get("head_dim") or H // c["num_attention_heads"],
        ffn=c["intermediate_size"], vocab=c["vocab_size"], norm_eps=float(c.get("rms_norm_eps", 1e-6)), act=act,
        rope_theta=float(full.get("rope_theta", 1000000.0)), rope_theta_local=float(local.get("rope_theta", 10000.0)),
        rope_proportion=float(full.get("partial_rotary_factor", 1.0)) if full.get("rope_type") == "proportional" else 1.0,
        max_position=int(c.get("max_position_embeddings", 131072)), tie_embeddings=bool(c.get("tie_word_embeddings", True)),
        layer_windows=[win if t == "sliding_attention" else 0 for t in lt], block="sandwich", qk_norm=True,
        final_softcap=float(cap) if cap else 0.0, embed_scale=float(H) ** 0.5,
        global_head_dim=int(c.get("global_head_dim") or 0), n_global_kv_heads=int(c.get("num_global_key_value_heads") or 0),
        k_eq_v=bool(c.get("attention_k_eq_v")), kv_shared_layers=int(c.get("num_kv_shared_layers") or 0),
        double_wide_mlp=bool(c.get("use_double_wide_mlp")), ple_dim=int(c.get("hidden_size_per_layer_input") or 0),
        ple_vocab=int(c.get("vocab_size_per_layer_input") or c["vocab_size"]), moe_block=moe,
        n_experts=int(c.get("num_experts") or 0) if moe else 0, top_k=int(c.get("top_k_experts") or 0) if moe else 0,
        moe_ffn=int(c.get("moe_intermediate_size") or 0) if moe else 0,
        bos_token=_token(c.get("bos_token_id"), 2), eos_token=_token(c.get("eos_token_id"), 1))


def _mpt(c):
    a = c.get("attn_config") or {}
    if not a.get("alibi", False):
        raise UnsupportedFamily("mpt without ALiBi (learned position table)")
    if a.get("clip_qkv") or a.get("qk_ln") or a.get("prefix_lm"):
        raise UnsupportedFamily("mpt with clip_qkv / qk_ln / prefix_lm")
    if not c.get("no_bias", True):
        raise UnsupportedFamily("mpt with biases")
    H, nh = c["d_model"], c["n_heads"]
    return DecoderConfig(name="mpt", family="mpt", n_layers=c["n_layers"], hidden=H, n_heads=nh, n_kv_heads=nh,
                         head_dim=H // nh, ffn=int(c.get("expansion_ratio", 4) * H), vocab=c["vocab_size"],
                         norm_eps=float(c.get("layer_norm_epsilon", 1e-5)), max_position=int(c.get("max_seq_len", 2048)),
                         tie_embeddings=True, norm_kind="layer", act="gelu_erf", gated_ffn=False, pos="alibi",
                         alibi_slopes="mpt", alibi_bias_max=float(a.get("alibi_bias_max", 8)),
                         attn_scale=a.get("softmax_scale"), logit_scale=float(c.get("logit_scale") or 1.0),
                         bos_token=_token(c.get("bos_token_id"), 0), eos_token=_token(c.get("eos_token_id"), 0))


def _bloom(c):
    if c.get("apply_residual_connection_post_layernorm"):
        raise UnsupportedFamily("bloom with the residual taken after the layer norm")
    H, nh = c["hidden_size"], c["n_head"]
    return DecoderConfig(name="bloom", family="bloom", n_layers=c["n_layer"], hidden=H, n_heads=nh, n_kv_heads=nh,
                         head_dim=H // nh, ffn=4 * H, vocab=c["vocab_size"], norm_eps=float(c.get("layer_norm_epsilon", 1e-5)),
                         max_position=int(c.get("seq_length", 2048)), tie_embeddings=True, norm_kind="layer",
                         norm_bias=True, embed_norm=True, act="gelu_tanh", gated_ffn=False, attn_bias=True, out_bias=True,
                         mlp_bias=True, pos="alibi", alibi_slopes="bloom",
                         bos_token=_token(c.get("bos_token_id"), 1), eos_token=_token(c.get("eos_token_id"), 2))


def _gpt_oss(c):
    return _base(c, "gpt_oss", attn_bias=True, out_bias=True, attn_sinks=True, n_experts=_experts(c),
                 top_k=c["num_experts_per_tok"], moe_ffn=c["intermediate_size"], router_bias=True, expert_bias=True,
                 swiglu_limit=float(c.get("swiglu_limit", 7.0)), norm_topk_prob=True)


def _minimax_m2(c):
    return _base(c, "minimax_m2", qk_norm=True, qk_norm_wide=True, n_experts=_experts(c), top_k=c["num_experts_per_tok"],
                 moe_ffn=c["intermediate_size"], router="sigmoid", router_select_bias=True, norm_topk_prob=True)


def _deepseek(c, family: str) -> DecoderConfig:
    rp = _rope_params(c)
    if (rp.get("rope_type") or rp.get("type") or "default") not in ("default", "none"):
        raise UnsupportedFamily(f"{family} with scaled rotary tables (the attention scale correction is not built)")
    dn, dr = c["qk_nope_head_dim"], c["qk_rope_head_dim"]
    v3 = family == "deepseek3"
    method = c.get("topk_method") or ("noaux_tc" if v3 else "greedy")
    if not v3 and method not in ("greedy",):
        raise UnsupportedFamily(f"deepseek2 routing method {method!r}")
    cfg = _base(c, family, kv_lora_rank=c["kv_lora_rank"], q_lora_rank=int(c.get("q_lora_rank") or 0), qk_nope_dim=dn,
                qk_rope_dim=dr, v_head_dim=c["v_head_dim"], head_dim=dn + dr, attn_scale=float(dn + dr) ** -0.5,
                rope_dim=None, rope_interleaved=bool(c.get("rope_interleave", True)), attn_bias=False, out_bias=False,
                n_experts=_experts(c), top_k=int(c.get("num_experts_per_tok") or 0),
                moe_ffn=int(c.get("moe_intermediate_size") or 0), n_shared_experts=int(c.get("n_shared_experts") or 0),
                first_dense_layers=int(c.get("first_k_dense_replace") or 0),
                routed_scale=float(c.get("routed_scaling_factor") or 1.0), norm_topk_prob=bool(c.get("norm_topk_prob", v3)))
    cfg.n_kv_heads = cfg.n_heads
    cfg.latent_norm_eps = 1e-6          # the norms of the low-rank query / key-value projections keep their own epsilon
    if v3:
        cfg.mtp_layers = int(c.get("num_nextn_predict_layers") or 0)     # used only when the checkpoint stores the layer
        cfg.router, cfg.router_select_bias = "sigmoid", True
        cfg.n_group, cfg.topk_group = int(c.get("n_group") or 1), int(c.get("topk_group") or 1)
    return cfg


def _with_indexer(cfg: DecoderConfig, c: dict) -> DecoderConfig:
    """Sparse attention fields of DeepSeek-V3.2 style headers (``index_topk`` / ``index_n_heads`` / ``index_head_dim``)."""
    cfg.index_topk, cfg.index_n_heads = int(c.get("index_topk") or 0), int(c.get("index_n_heads") or 0)
    cfg.index_head_dim = int(c.get("index_head_dim") or 0)
    if cfg.index_topk and not cfg.q_lora_rank:
        raise UnsupportedFamily("a sparse attention indexer needs the low-rank query projection it reads")
    if cfg.index_topk and cfg.index_head_dim < cfg.qk_rope_dim:
        raise UnsupportedFamily("indexer heads narrower than the rotary part")
    return cfg


def _deepseek32(c):
    cfg = _with_indexer(_deepseek(c, "deepseek3"), c)
    cfg.family = "deepseek32"
    return cfg


def _glm_moe_dsa(c):
    """GLM with latent attention and the sparse attention indexer: DeepSeek-V3 style stack, half-split rotary, dense or
    routed FFN by ``mlp_layer_types``."""
    cfg = _with_indexer(_deepseek({**c, "rope_interleave": False, "first_k_dense_replace": 0}, "deepseek3"), c)
    cfg.family = "glm_moe_dsa"
    kinds = list(c.get("mlp_layer_types") or [])[:cfg.n_layers]
    cfg.dense_layers = [i for i, k in enumerate(kinds) if k == "dense"] or None
    return cfg


def _glm53(c):
    """GLM-5.3-Flash (``glm5_next``: the text tower's header sits under ``text_config``; crates/poot-models/src/
    architectures/glm53_flash/config.rs).  What the tracer does not implement is refused by name, not assumed."""
    from .glm53 import Glm53Config
    t = dict(c.get("text_config") or {})
    if not t:
        raise UnsupportedFamily("glm5_next header without text_config")
    for k in ("eos_token_id", "bos_token_id", "tie_word_embeddings"):
        if c.get(k) is not None:
            t[k] = c[k]
    for key, accepted in (("hidden_act", ("silu",)), ("scoring_func", ("sigmoid",)), ("topk_method", ("noaux_tc",))):
        if t.get(key) is not None and t[key] not in accepted:
            raise UnsupportedFamily(f"glm5_next {key} {t[key]!r}")
    for key, supported in (("mla_use_nope", True), ("index_kpool_compress", True), ("index_kpool_always_select_tail", True),
                           ("attention_bias", False)):
        if t.get(key) is not None and bool(t[key]) != supported:
            raise UnsupportedFamily(f"glm5_next with {key}={t[key]!r}")
    L, H = int(t["num_hidden_layers"]), int(t["hidden_size"])
    kinds = [{"linear_attention": "kda", "deepseek_sparse_attention": "dsa"}.get(k) for k in (t.get("layer_types") or [])]
    ffns = list(t.get("mlp_layer_types") or [])
    if len(kinds) != L or None in kinds or len(ffns) != L or any(f not in ("dense", "sparse") for f in ffns):
        raise UnsupportedFamily(f"glm5_next layer schedule {t.get('layer_types')!r} / {t.get('mlp_layer_types')!r} for {L} layers")
    mtp = int(t.get("num_nextn_predict_layers") or 0)
    has_dsa = "dsa" in kinds or mtp > 0
    if has_dsa and int(t.get("qk_rope_head_dim") or 0) != 0:
        raise UnsupportedFamily("glm5_next with a rotary part in its latent attention")
    if has_dsa and any(x != "full" for x in (t.get("indexer_types") or [])):
        raise UnsupportedFamily(f"glm5_next indexer types {t.get('indexer_types')!r}")
    lin = dict(t.get("linear_attn_config") or {})
    if "kda" in kinds and not all(k in lin for k in ("num_heads", "head_dim", "short_conv_kernel_size", "gate_lower_bound")):
        raise UnsupportedFamily("glm5_next linear-attention layers without a complete linear_attn_config")
    lower = float(lin.get("gate_lower_bound", -5.0))
    if not lower < 0:
        raise UnsupportedFamily(f"glm5_next gate_lower_bound {lower}")
    pool, topk = int(t.get("index_kpool") or 1), int(t.get("index_topk") or 0)
    if has_dsa and (topk < 1 or topk % pool):
        raise UnsupportedFamily(f"glm5_next index_topk {topk} is not a positive multiple of index_kpool {pool}")
    sparse = "sparse" in ffns
    inter = int(t.get("moe_intermediate_size") or 0)
    return Glm53Config(
        name="glm53_flash", family="glm53_flash", n_layers=L, hidden=H, n_heads=int(t.get("num_attention_heads") or 1),
        n_kv_heads=int(t.get("num_attention_heads") or 1), head_dim=int(t.get("qk_nope_head_dim") or 0) or 1,
        ffn=int(t.get("intermediate_size") or 0), vocab=int(t["vocab_size"]), norm_eps=float(t.get("rms_norm_eps", 1e-5)),
        max_position=int(t["max_position_embeddings"]), tie_embeddings=bool(t.get("tie_word_embeddings", False)), pos="none",
        layer_kinds=kinds, ffn_kinds=ffns, hc_mult=int(t["hc_mult"]), hc_eps=float(t.get("hc_eps", 1e-6)),
        hc_iters=int(t["hc_sinkhorn_iters"]), kda_heads=int(lin.get("num_heads") or 0), kda_head_dim=int(lin.get("head_dim") or 0),
        kda_conv=int(lin.get("short_conv_kernel_size") or 4), kda_lower_bound=lower,
        q_lora_rank=int(t.get("q_lora_rank") or 0), kv_lora_rank=int(t.get("kv_lora_rank") or 0),
        qk_nope_dim=int(t.get("qk_nope_head_dim") or 0), v_head_dim=int(t.get("v_head_dim") or 0),
        index_n_heads=int(t.get("index_n_heads") or 0), index_head_dim=int(t.get("index_head_dim") or 0), index_topk=topk,
        index_kpool=pool, n_experts=int(t.get("n_routed_experts") or 0) if sparse else 0,
        top_k=int(t.get("num_experts_per_tok") or 0), moe_ffn=inter, n_shared_experts=int(t.get("n_shared_experts", 1)),
        n_group=int(t.get("n_group") or 1), topk_group=int(t.get("topk_group") or 1),
        routed_scale=float(t.get("routed_scaling_factor", 1.0)), norm_topk_prob=bool(t.get("norm_topk_prob", True)),
        router="sigmoid", router_select_bias=True, swiglu_limit=float(t.get("swiglu_limit", 10.0)), mtp_layers=mtp,
        bos_token=_token(t.get("bos_token_id"), 1), eos_token=_token(t.get("eos_token_id"), 2))


def _deepseek4(c):
    """DeepSeek-V4 (``deepseek_v4``; crates/poot-models/src/architectures/deepseek4/config.rs).  The layer kinds come
    from ``compress_ratios`` (0: window only; the sparse rate; the heavy rate); a router or a rotary scaling the tracer
    does not implement is refused by name."""
    from .deepseek4 import DeepseekV4Config
    if c.get("scoring_func") not in (None, "sqrtsoftplus"):
        raise UnsupportedFamily(f"deepseek_v4 scoring_func {c.get('scoring_func')!r}")
    rs = c.get("rope_scaling") or {}
    if (rs.get("rope_type") or rs.get("type") or "default") not in ("default", "none"):
        raise UnsupportedFamily(f"deepseek_v4 rope_scaling {rs!r}")
    L, H, nh, D = int(c["num_hidden_layers"]), int(c["hidden_size"]), int(c["num_attention_heads"]), int(c["head_dim"])
    rot, groups = int(c["qk_rope_head_dim"]), int(c["o_groups"])
    if rot > D or rot % 2:
        raise UnsupportedFamily(f"deepseek_v4 qk_rope_head_dim {rot} for heads of {D}")
    if (nh * D) % groups:
        raise UnsupportedFamily(f"deepseek_v4 o_groups {groups} does not divide {nh * D}")
    rates = dict(c.get("compress_rates") or {})
    csa, hca = int(rates.get("compressed_sparse_attention", 4)), int(rates.get("heavily_compressed_attention", 128))
    if csa < 1 or hca < 1 or csa == hca:
        raise UnsupportedFamily(f"deepseek_v4 compress_rates {rates!r}")
    ratios = list(c.get("compress_ratios") or [])
    if len(ratios) < L:
        raise UnsupportedFamily(f"deepseek_v4 compress_ratios names {len(ratios)} of {L} layers")
    kinds = [{0: "sliding", csa: "csa", hca: "hca"}.get(int(r)) for r in ratios[:L]]
    if None in kinds:
        raise UnsupportedFamily(f"deepseek_v4 compress_ratios {ratios[:L]!r} outside 0 / {csa} / {hca}")
    ni, di, topk = int(c.get("index_n_heads") or 0), int(c.get("index_head_dim") or 0), int(c.get("index_topk") or 0)
    if "csa" in kinds and (ni < 1 or topk < 1 or di < rot):
        raise UnsupportedFamily(f"deepseek_v4 indexer of {ni} heads of {di} keeping {topk}")
    hashed = int(c.get("num_hash_layers") or 0)
    if hashed > L:
        raise UnsupportedFamily(f"deepseek_v4 num_hash_layers {hashed} exceeds {L} layers")
    return DeepseekV4Config(
        name="deepseek4", family="deepseek4", n_layers=L, hidden=H, n_heads=nh, n_kv_heads=1, head_dim=D, ffn=0,
        vocab=int(c["vocab_size"]), norm_eps=float(c.get("rms_norm_eps", 1e-6)), max_position=int(c["max_position_embeddings"]),
        rope_theta=float(c.get("rope_theta", 10000.0)), compress_rope_theta=float(c.get("compress_rope_theta", 160000.0)),
        qk_rope_dim=rot, q_lora_rank=int(c["q_lora_rank"]), o_groups=groups, o_lora_rank=int(c["o_lora_rank"]),
        sliding_window=int(c["sliding_window"]), attn_kinds=kinds, csa_rate=csa, hca_rate=hca, index_n_heads=ni, index_head_dim=di,
        index_topk=topk, hc_mult=int(c["hc_mult"]), hc_eps=float(c.get("hc_eps", 1e-6)), hc_iters=int(c["hc_sinkhorn_iters"]),
        n_experts=int(c["n_routed_experts"]), top_k=int(c["num_experts_per_tok"]), moe_ffn=int(c["moe_intermediate_size"]),
        n_shared_experts=int(c.get("n_shared_experts", 1)), routed_scale=float(c.get("routed_scaling_factor", 1.0)),
        router="sqrtsoftplus", router_select_bias=True, swiglu_limit=float(c.get("swiglu_limit", 10.0)), hash_layers=hashed,
        attn_sinks=True, pos="rope", bos_token=_token(c.get("bos_token_id"), 1), eos_token=_token(c.get("eos_token_id"), 2))


def _deepseek2(c): return _deepseek(c, "deepseek2")
def _deepseek3(c): return _deepseek(c, "deepseek3")


def _nemotron_h(c):
    kinds = c.get("layers_block_type") or c.get("layer_types")
    if not kinds and c.get("hybrid_override_pattern"):
        kinds = [{"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}[ch] for ch in c["hybrid_override_pattern"]]
    if not kinds:
        raise UnsupportedFamily("nemotron_h header without a block pattern")
    if c.get("moe_latent_size"):
        raise UnsupportedFamily("nemotron_h with a latent expert projection")
    H, nh = c["hidden_size"], c["num_attention_heads"]
    def _num(v, default):      # JSON has no infinity: writers spell it as a string or a tagged object
        if isinstance(v, (int, float)):
            return float(v)
        if isinstance(v, dict):
            v = v.get("__float__")
        if isinstance(v, str):
            return float(v.replace("Infinity", "inf"))
        return default
    lim = c.get("time_step_limit") or [0.0, float("inf")]
    if _num(lim[0], 0.0) > 0.0 or _num(lim[1], float("inf")) != float("inf"):
        raise UnsupportedFamily("nemotron_h with a clamped time step")
    act = {"relu2": "relu2", "silu": "silu", "gelu": "gelu_erf"}.get(c.get("mlp_hidden_act", "relu2"))
    if act is None:
        raise UnsupportedFamily(f"nemotron_h activation {c.get('mlp_hidden_act')!r}")
    moe = any(k == "moe" for k in kinds)
    cfg = DecoderConfig(
        name="nemotron_h", family="nemotron_h", n_layers=len(kinds), hidden=H, n_heads=nh,
        n_kv_heads=c.get("num_key_value_heads") or nh, head_dim=c.get("head_dim") or H // nh, ffn=c.get("intermediate_size", 4 * H),
        vocab=c["vocab_size"], norm_eps=float(c.get("layer_norm_epsilon", 1e-5)), pos="none",
        max_position=int(c.get("max_position_embeddings", 4096)), tie_embeddings=bool(c.get("tie_word_embeddings", False)),
        act=act, gated_ffn=False, mlp_bias=bool(c.get("mlp_bias", False)),
        layer_kinds=[k if k in ("mamba", "attention") else "none" for k in kinds],
        layer_ffn=[int(k in ("mlp", "moe")) for k in kinds],
        dense_layers=[i for i, k in enumerate(kinds) if k == "mlp"],
        ssm_heads=c["mamba_num_heads"], ssm_head_dim=c["mamba_head_dim"], ssm_state=c["ssm_state_size"],
        ssm_groups=c.get("n_groups", 1), ssm_conv=c.get("conv_kernel", 4), ssm_conv_bias=bool(c.get("use_conv_bias", True)),
        bos_token=_token(c.get("bos_token_id"), 1), eos_token=_token(c.get("eos_token_id"), 2))
    if c.get("attention_bias") or c.get("use_bias"):
        raise UnsupportedFamily("nemotron_h with projection biases")
    if moe:
        cfg.n_experts, cfg.top_k, cfg.moe_ffn = _experts(c), c["num_experts_per_tok"], c["moe_intermediate_size"]
        cfg.router, cfg.router_select_bias = "sigmoid", True
        cfg.n_group, cfg.topk_group = int(c.get("n_group") or 1), int(c.get("topk_group") or 1)
        cfg.norm_topk_prob = bool(c.get("norm_topk_prob", True))
        cfg.routed_scale = float(c.get("routed_scaling_factor") or 1.0)
        cfg.shared_ffn = int(c.get("moe_shared_expert_intermediate_size") or 0)
    return cfg


def _qwen3next(c):
    kinds = c.get("layer_types")
    L = c["num_hidden_layers"]
    if not kinds:
        every = int(c.get("full_attention_interval") or 4)
        kinds = ["full_attention" if (i + 1) % every == 0 else "linear_attention" for i in range(L)]
    if c["linear_key_head_dim"] != c["linear_value_head_dim"]:
        raise UnsupportedFamily("qwen3_next with different key and value head widths in the delta-net layers")
    step = int(c.get("decoder_sparse_step") or 1)
    only = set(c.get("mlp_only_layers") or [])
    E = _experts(c)
    cfg = _base({**c, "layer_types": None}, "qwen3next", qk_norm=True, out_bias=False, attn_gate=True, norm_offset=1.0,
                layer_kinds=["attention" if k == "full_attention" else "gdn" for k in kinds],
                gdn_k_heads=c["linear_num_key_heads"], gdn_v_heads=c["linear_num_value_heads"],
                gdn_head_dim=c["linear_key_head_dim"], gdn_conv=c.get("linear_conv_kernel_dim", 4),
                n_experts=E, top_k=int(c.get("num_experts_per_tok") or 0), moe_ffn=int(c.get("moe_intermediate_size") or 0),
                norm_topk_prob=bool(c.get("norm_topk_prob", True)),
                shared_ffn=int(c.get("shared_expert_intermediate_size") or 0) if E else 0, shared_expert_gate=bool(E),
                dense_layers=[i for i in range(L) if E and (i in only or (i + 1) % step != 0)] or None)
    return cfg


def _qwen35(c):
    """Qwen3.5 text tower (``qwen3_5_text``, or ``qwen3_5`` with the tower's header nested under ``text_config``): the
    Qwen3-Next body with a dense gated FFN where Qwen3-Next routes (architectures/qwen38_27b.rs:1-12)."""
    c = c.get("text_config") or c
    cfg = _qwen3next(c)
    cfg.family = "qwen38_27b"
    return cfg


def _qwen38(c):
    """Qwen3.8-Flash-Next (``qwen4_exp``; crates/poot-models/src/architectures/qwen38/config.rs): the Qwen3-Next layer
    (gated delta net or gated attention, routed experts with a gated shared expert) inside gated hyper-connections,
    with a block indexer narrowing the full-attention layers and hashed n-gram embedding blocks in front of the layers
    ``ple_layer_ids`` names (1-based)."""
    t = dict(c.get("text_config") or {})
    if not t:
        raise UnsupportedFamily("qwen4_exp header without text_config")
    for k in ("eos_token_id", "bos_token_id", "tie_word_embeddings"):
        if k not in t and c.get(k) is not None:
            t[k] = c[k]
    for flag in ("attention_bias", "use_sliding_window"):
        if t.get(flag):
            raise UnsupportedFamily(f"qwen4_exp with {flag}")
    if not t.get("layer_types") or len(t["layer_types"]) != t["num_hidden_layers"]:
        raise UnsupportedFamily("qwen4_exp header without one layer_types entry per layer")
    if t.get("partial_rotary_factor") is None:
        raise UnsupportedFamily("qwen4_exp header without partial_rotary_factor")
    if int(t.get("indexer_kv_heads", 1)) != 1:
        raise UnsupportedFamily("qwen4_exp indexer_kv_heads other than 1 (the indexer shares one key per token)")
    gate = t.get("output_gate_type") or t.get("hidden_act") or "silu"
    if gate not in ("silu", "sigmoid"):
        raise UnsupportedFamily(f"qwen4_exp output_gate_type {gate!r}")
    cfg = _qwen3next(t)
    ratio, budget = int(t.get("indexer_compress_ratio") or 0), int(t.get("indexer_budget") or 0)
    ni, di = int(t.get("indexer_n_heads") or 0), int(t.get("indexer_head_dim") or 0)
    if "attention" in cfg.layer_kinds:
        if ratio < 1 or ratio & (ratio - 1):
            raise UnsupportedFamily(f"qwen4_exp indexer_compress_ratio {ratio} is not a power of two")
        if budget < ratio or ni < 1 or di < cfg.rot:
            raise UnsupportedFamily(f"qwen4_exp indexer of {ni} heads of {di} with a budget of {budget} over blocks of {ratio}")
    ids = list(t.get("ple_layer_ids") or [])
    layers = [int(i) - 1 for i in ids]
    if any(not 0 <= l < cfg.n_layers or cfg.layer_kinds[l] != "gdn" for l in layers) or len(set(layers)) != len(layers):
        raise UnsupportedFamily(f"qwen4_exp ple_layer_ids {ids!r}: distinct linear-attention layers, counted from 1")
    if layers:
        n, per, emb = int(t.get("ngram_size") or 0), int(t.get("heads_per_ngram") or 0), int(t.get("ple_embed_dim") or 0)
        if n not in (2, 3) or per < 1 or emb < 1 or emb % ((n - 1) * per) or int(t.get("ple_conv_kernel_size") or 0) < 2:
            raise UnsupportedFamily(f"qwen4_exp n-gram block: order {n}, {per} heads per order, embedding {emb}, "
                                    f"conv {t.get('ple_conv_kernel_size')}")
        if t.get("ngram_vocab_size_base") is None:
            raise UnsupportedFamily("qwen4_exp header without ngram_vocab_size_base")
    streams, rank = int(t.get("hc_count") or 0), int(t.get("hc_lowrank") or 0)
    if streams < 1 or rank < 1:
        raise UnsupportedFamily(f"qwen4_exp hc_count {streams} / hc_lowrank {rank}")
    cfg.family = cfg.name = "qwen38"
    cfg.hc_count, cfg.hc_lowrank, cfg.gdn_gate_act = streams, rank, gate
    cfg.index_ratio, cfg.index_budget, cfg.index_n_heads, cfg.index_head_dim = ratio, budget, ni, di
    cfg.ple_layers = layers or None
    if layers:
        cfg.ple_embed_dim, cfg.ple_conv, cfg.ngram_size, cfg.heads_per_ngram = emb, int(t["ple_conv_kernel_size"]), n, per
        cfg.ngram_vocab_base, cfg.ngram_divisible_by = int(t["ngram_vocab_size_base"]), int(t.get("make_ngram_vocab_size_divisible_by") or 1)
        cfg.ngram_seed = int(t.get("seed", 1234))
    return cfg


def _idefics3(c):
    """Idefics3 / SmolVLM: a llama text stack behind a SigLIP-style vision tower and a pixel-shuffle connector."""
    from .vision import VisionConfig
    t, v = dict(c.get("text_config") or {}), dict(c.get("vision_config") or {})
    if (t.get("model_type") or "llama") != "llama":
        raise UnsupportedFamily(f"idefics3 over a {t.get('model_type')!r} text stack")
    t.setdefault("tie_word_embeddings", c.get("tie_word_embeddings", False))
    text = _llama(t)
    text.family = "idefics3"
    act = {"gelu_pytorch_tanh": "gelu_tanh", "gelu_new": "gelu_tanh", "gelu": "gelu_erf"}.get(v.get("hidden_act", "gelu_pytorch_tanh"))
    if act is None:
        raise UnsupportedFamily(f"idefics3 vision activation {v.get('hidden_act')!r}")
    vision = VisionConfig(hidden=v.get("hidden_size", 1152), ffn=v.get("intermediate_size", 3072),
                          n_layers=v.get("num_hidden_layers", 12), n_heads=v.get("num_attention_heads", 16),
                          channels=v.get("num_channels", 3), image_size=v.get("image_size", 224), patch=v.get("patch_size", 32),
                          norm_eps=float(v.get("layer_norm_eps", 1e-6)), act=act, scale=int(c.get("scale_factor", 2)),
                          text_hidden=text.hidden)
    if vision.per_side % vision.scale:
        raise UnsupportedFamily(f"idefics3: {vision.per_side} patches per side do not fold by {vision.scale}")
    return text, vision, int(c.get("image_token_id", 128257))


def _qwen_vl(c):
    """Qwen2.5-VL: a Qwen2 text stack with sectioned rotary positions behind a windowed-attention vision tower."""
    from .vision import QwenVisionConfig
    t = dict(c.get("text_config") or c)
    v = dict(c.get("vision_config") or {})
    t.setdefault("tie_word_embeddings", c.get("tie_word_embeddings", False))
    rp = t.get("rope_parameters") or t.get("rope_scaling") or {}
    sections = rp.get("mrope_section")
    if not sections:
        raise UnsupportedFamily("qwen2_5_vl header without mrope_section")
    plain = {k: x for k, x in t.items() if k not in ("rope_scaling", "rope_parameters")}
    plain["rope_theta"] = rp.get("rope_theta", t.get("rope_theta", 1000000.0))
    plain["use_sliding_window"] = False
    text = _base(plain, "qwen_vl", attn_bias=True, out_bias=False)
    text.mrope_sections = [int(x) for x in sections]
    act = {"silu": "silu", "gelu_pytorch_tanh": "gelu_tanh", "gelu": "gelu_erf"}.get(v.get("hidden_act", "silu"))
    if act is None:
        raise UnsupportedFamily(f"qwen2_5_vl vision activation {v.get('hidden_act')!r}")
    vision = QwenVisionConfig(hidden=v.get("hidden_size", 1280), ffn=v.get("intermediate_size", 3420), n_layers=v.get("depth", 32),
                              n_heads=v.get("num_heads", 16), channels=v.get("in_channels", v.get("in_chans", 3)),
                              patch=v.get("patch_size", 14), temporal=v.get("temporal_patch_size", 2),
                              merge=v.get("spatial_merge_size", 2), window=v.get("window_size", 112),
                              full_layers=tuple(v.get("fullatt_block_indexes", (7, 15, 23, 31))),
                              out_hidden=v.get("out_hidden_size", text.hidden), act=act,
                              video_token=int(c.get("video_token_id", -1)), tokens_per_second=float(v.get("tokens_per_second", 2)))
    if vision.out_hidden != text.hidden:
        raise UnsupportedFamily("qwen2_5_vl: the merger's output width differs from the text width")
    return text, vision, int(c.get("image_token_id", 151655))


def _bert(c):
    from .encoder import EncoderConfig
    if (c.get("position_embedding_type") or "absolute") != "absolute":
        raise UnsupportedFamily("bert with relative position embeddings")
    act = {"gelu": "gelu_erf", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "relu": "relu"}.get(c.get("hidden_act", "gelu"))
    if act is None:
        raise UnsupportedFamily(f"bert activation {c.get('hidden_act')!r}")
    arch = " ".join(c.get("architectures") or [])
    labels = len(c.get("id2label") or {}) or int(c.get("num_labels") or 0) if "SequenceClassification" in arch else 0
    return EncoderConfig(n_layers=c["num_hidden_layers"], hidden=c["hidden_size"], n_heads=c["num_attention_heads"],
                         ffn=c["intermediate_size"], vocab=c["vocab_size"], max_position=c.get("max_position_embeddings", 512),
                         type_vocab=c.get("type_vocab_size", 2), norm_eps=float(c.get("layer_norm_eps", 1e-12)), act=act,
                         labels=labels, pad_token=int(c.get("pad_token_id") or 0))


SHIPPED: List[FamilyEntry] = [
    FamilyEntry("qwen2", ["qwen2"], ["qwen2"], _qwen2),
    FamilyEntry("llama", ["llama", "mistral", "mixtral"], ["llama"], _llama),
    FamilyEntry("qwen3", ["qwen3"], ["qwen3"], _qwen3),
    FamilyEntry("olmo2", ["olmo2"], ["olmo2"], _olmo2),
    FamilyEntry("phi3", ["phi3"], ["phi3"], _phi3),
    FamilyEntry("smollm3", ["smollm3"], ["smollm3"], _smollm3),
    FamilyEntry("granite", ["granite", "granitemoe"], ["granite", "granitemoe"], _granite),
    FamilyEntry("mpt", ["mpt"], ["mpt"], _mpt),
    FamilyEntry("bloom", ["bloom"], ["bloom"], _bloom),
    FamilyEntry("gemma3", ["gemma3", "gemma3_text"], ["gemma3"], _gemma3),
    FamilyEntry("gemma2", ["gemma2"], ["gemma2"], _gemma2),
    FamilyEntry("gemma4", ["gemma4", "gemma4_text"], ["gemma4"], _gemma4, kind="own", tracer="gemma4:Gemma4Model"),
    FamilyEntry("qwen3moe", ["qwen3_moe"], ["qwen3moe"], _qwen3moe),
    FamilyEntry("gpt_oss", ["gpt_oss"], ["gpt-oss"], _gpt_oss),
    FamilyEntry("olmoe", ["olmoe"], ["olmoe"], _olmoe),
    FamilyEntry("minimax_m2", ["minimax_m2"], ["minimax-m2"], _minimax_m2),
    FamilyEntry("deepseek2", ["deepseek_v2"], ["deepseek2"], _deepseek2),
    FamilyEntry("deepseek3", ["deepseek_v3"], ["deepseek2"], _deepseek3),
    FamilyEntry("deepseek32", ["deepseek_v32"], ["deepseek32"], _deepseek32),
    FamilyEntry("glm_moe_dsa", ["glm_moe_dsa"], [], _glm_moe_dsa),
    FamilyEntry("nemotron_h", ["nemotron_h"], ["nemotron_h"], _nemotron_h),
    FamilyEntry("qwen3next", ["qwen3_next"], ["qwen3next"], _qwen3next),
    FamilyEntry("qwen38_27b", ["qwen3_5", "qwen3_5_text"], ["qwen35"], _qwen35),
    FamilyEntry("bert", ["bert"], ["bert"], _bert, kind="encoder"),
    FamilyEntry("idefics3", ["idefics3", "smolvlm"], [], _idefics3, kind="vlm"),
    FamilyEntry("qwen_vl", ["qwen2_5_vl"], [], _qwen_vl, kind="vlm"),
    FamilyEntry("glm53_flash", ["glm5_next"], [], _glm53, kind="own", tracer="glm53:Glm53Model"),
    FamilyEntry("deepseek4", ["deepseek_v4"], [], _deepseek4, kind="own", tracer="deepseek4:DeepseekV4Model"),
    FamilyEntry("qwen38", ["qwen4_exp"], [], _qwen38),
]


# families whose GGUF metadata and tensor names the generic llama-style reader covers completely
GGUF_FAMILIES = ("llama", "qwen2", "qwen3", "qwen3moe", "phi3", "olmo2", "olmoe", "smollm3", "granite", "gemma2", "gemma3", "gpt_oss",
                 "mpt", "bloom", "minimax_m2", "deepseek2", "qwen38_27b", "gemma4")
# of those, the ones whose configuration is read by the family's own header table from a header rebuilt out of the GGUF keys
GGUF_VIA_HEADER = ("olmo2", "olmoe", "smollm3", "granite", "gemma2", "gemma3", "gpt_oss", "mpt", "bloom", "minimax_m2", "deepseek2", "qwen38_27b", "gemma4")


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
                if e.kind == "encoder":
                    from .encoder import EncoderModel
                    return EncoderModel(e.from_hf(config))
                if e.kind == "own":
                    import importlib
                    mod, cls = e.tracer.split(":")
                    return getattr(importlib.import_module("." + mod, __package__), cls)(e.from_hf(config))
                if e.kind == "vlm":
                    from .vision import QwenVisionConfig, QwenVisionTower, VisionLanguageModel, VisionTower
                    text, vision, image_token = e.from_hf(config)
                    tower = QwenVisionTower(vision) if isinstance(vision, QwenVisionConfig) else VisionTower(vision)
                    return VisionLanguageModel(Model(text), tower, image_token)
                return Model(e.from_hf(config))
        raise UnsupportedFamily(f"no family for model_type {mt!r}")

    def resolve_gguf(self, arch: str, meta: dict) -> Model:
        from ..load.gguf import config_from_gguf_metadata
        for e in self.entries:
            if arch in e.gguf_archs:
                if e.from_hf is None:
                    raise UnsupportedFamily(f"family {e.name!r} needs {e.missing}, which this build does not have")
                if e.name not in GGUF_FAMILIES:
                    # the GGUF header of these families carries fields (norm placement, soft caps, window patterns,
                    # multipliers, router kinds) that only their Hugging Face header table reads here
                    raise UnsupportedFamily(f"family {e.name!r}: no GGUF header / tensor-name table; load the Hugging Face "
                                            "checkpoint directory (config.json + safetensors) instead")
                if e.name in GGUF_VIA_HEADER:
                    from ..load.gguf import hf_header_from_gguf
                    cfg = e.from_hf(hf_header_from_gguf(arch, meta, e.name))
                    cfg.name = str(meta.get("general.name", e.name))
                    if e.name in ("gemma2", "gemma3", "qwen38_27b"):
                        cfg.norm_offset = 0.0           # llama.cpp's converter stores these norm scales with the one folded in
                    if e.kind == "own":
                        import importlib
                        mod, cls = e.tracer.split(":")
                        return getattr(importlib.import_module("." + mod, __package__), cls)(cfg)
                    return Model(cfg)
                return Model(config_from_gguf_metadata(arch, meta, e.name))
        raise UnsupportedFamily(f"no family for GGUF architecture {arch!r}")

    def supported(self) -> List[str]:
        return [e.name for e in self.entries if e.from_hf is not None]

    def listed(self) -> List[str]:
        return [e.name for e in self.entries]
