"""Model trait, step specification and the shared "standard stack" tracer.

A model is a function that traces one *step* into the graph IR (crates/poot-models/src/model.rs:189-417):
``StepSpec`` fixes the static shapes (rows, tokens per row, KV capacity, KV layout, which rows get logits) and
the tracer records embed -> layers of ``x += mixer(norm(x)); x += ffn(norm(x))`` -> final norm -> head
(crates/poot-models/src/components/standard.rs:618-866).  The KV write is a paged ``scatter_update`` through the
write map followed by ``paged_view`` through the read map, or a contiguous ``dynamic_update_slice``
(components/attention.rs:453-533).  Family modules only provide a ``DecoderConfig`` and weight-name tables.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

from ..ir import oplib as O
from ..ir.builder import Builder, Traced
from ..ir.graph import Graph
from ..tensor import DType
from .config import DecoderConfig

F32, I32 = DType.F32, DType.I32


@dataclass(frozen=True)
class StepSpec:
    rows: int = 1                 # sequences in the step
    tokens: int = 1               # tokens per row (1 = decode, >1 = prefill chunk)
    capacity: int = 64            # KV positions visible to a row
    paged: bool = True
    pool_slots: int = 0           # paged: slots in each layer's pool (0 -> rows * capacity)
    logit_rows: str = "last"      # last | all
    kv_dtype: DType = DType.F32
    weight_dtype: DType = DType.F32
    sampler: Optional[str] = None  # None = export logits; greedy | gumbel | gumbel_top_k | gumbel_top_k_top_p
    world: int = 1                # tensor-parallel world (the tracer emits all_reduce at the Megatron points)
    carry: bool = False           # also export the closing-norm hidden state of the logit rows ("hidden"): what a
    #                               multi-token-prediction layer reads and a chain of its steps recycles
    embeds: bool = False          # rows of other modalities replace the embeddings of flagged tokens (image rows of a VLM)
    mrope: bool = False           # three rotary position streams (time, row, column) bind per token: ``rope_positions[3, R*T]``
    gdn_chunk: int = 0            # > 0: steps of more than one token run the gated delta rule in its chunk-parallel form
    #                               (matrix products over chunks of this many tokens) instead of the per-token scan equation
    weight_formats: tuple = ()    # ((weight name, block format), ..): those 2-D weights are declared as their packed bytes and
    #                               decoded by a ``packed_dequant`` equation, so an evaluator or a planner sees them as stored

    @property
    def slots(self) -> int:
        return self.pool_slots or self.rows * self.capacity


def spec_rank_heads(spec: StepSpec, heads_per_rank: int) -> slice:
    """Heads a trace covers (the tracer has no rank of its own: a sharded trace describes rank 0's share)."""
    return slice(0, heads_per_rank)


class Model:
    """One loaded architecture: configuration + tracer + weight-name tables."""

    def __init__(self, cfg: DecoderConfig):
        self.cfg = cfg

    def mtp_model(self) -> "Model":
        """The checkpoint's multi-token-prediction layer as a one-block model of its own."""
        from .config import mtp_config
        return type(self)(mtp_config(self.cfg))

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H, D = c.hidden, c.head_dim
        s = {"embed": (c.vocab, H), "final_norm": (H,)}
        norms = ["final_norm"]
        S = c.hc_count
        if S:
            # gated hyper-connections: no plain norms; every gate has a grouped norm scale, a low-rank gate and, inside
            # a layer, the per-stream injection projection; the closing gate collapses the streams into the head
            del s["final_norm"]
            norms = []
            gate = lambda stem, inject: {stem + "norm": (S * H,), stem + "down": (c.hc_lowrank, S * H), stem + "up": (S * H, c.hc_lowrank),
                                         **({stem + "inject": (S, S * H)} if inject else {})}
            s.update(gate("hc_final_", False))
        if c.embed_norm:
            s["embed_norm"] = (H,)
            norms.append("embed_norm")
        if not c.tie_embeddings:
            s["lm_head"] = (c.vocab, H)
        if c.mtp_head:
            s.update({"mtp.enorm": (H,), "mtp.hnorm": (H,), "mtp.eh_proj": (H, 2 * H)})
            norms += ["mtp.enorm", "mtp.hnorm"]
        for l in range(c.n_layers):
            p = f"layers.{l}."
            kind, has_ffn = c.mixer_of(l), c.has_ffn(l)
            if S:
                s.update(gate(p + "hc_attn_", True))
                s.update(gate(p + "hc_ffn_", True))
                t_ = c.ple_tables(l)
                if t_ is not None:
                    s.update({p + "ple_table": (t_.rows, c.ple_embed_dim // len(t_.primes)), p + "ple_key": (S * H, c.ple_embed_dim),
                              p + "ple_value": (H, c.ple_embed_dim), p + "ple_key_norm": (S * H,), p + "ple_query_norm": (S * H,),
                              p + "ple_conv_norm": (S * H,), p + "ple_conv": (S * H, c.ple_conv)})
            elif c.block in ("pre", "sandwich"):
                if kind != "none":
                    s[p + "attn_norm"] = (H,)
                    norms.append(p + "attn_norm")
                if has_ffn:
                    s[p + "ffn_norm"] = (H,)
                    norms.append(p + "ffn_norm")
            if c.block in ("post", "sandwich"):
                s[p + "attn_post_norm"] = (H,)
                s[p + "ffn_post_norm"] = (H,)
                norms += [p + "attn_post_norm", p + "ffn_post_norm"]
            if kind == "mamba":
                I, G, N = c.ssm_heads * c.ssm_head_dim, c.ssm_groups, c.ssm_state
                C = I + 2 * G * N
                s.update({p + "ssm_in_z": (I, H), p + "ssm_in_x": (C, H), p + "ssm_in_dt": (c.ssm_heads, H),
                          p + "ssm_conv": (C, c.ssm_conv), p + "ssm_dt_bias": (c.ssm_heads,), p + "ssm_a_log": (c.ssm_heads,),
                          p + "ssm_d": (c.ssm_heads,), p + "ssm_gate_norm_w": (I,), p + "ssm_o": (H, I)})
                if c.ssm_conv_bias:
                    s[p + "ssm_conv_bias"] = (C,)
            elif kind == "gdn":
                nk, nv, Dg = c.gdn_k_heads, c.gdn_v_heads, c.gdn_head_dim
                s.update({p + "gdn_q": (nk * Dg, H), p + "gdn_k": (nk * Dg, H), p + "gdn_v": (nv * Dg, H),
                          p + "gdn_z": (nv * Dg, H), p + "gdn_b": (nv, H), p + "gdn_a": (nv, H),
                          p + "gdn_conv": ((2 * nk + nv) * Dg, c.gdn_conv), p + "gdn_dt_bias": (nv,), p + "gdn_a_log": (nv,),
                          p + "gdn_gate_norm_w": (Dg,), p + "gdn_o": (H, nv * Dg)})
            elif kind == "attention" and c.is_mla:
                qk = c.qk_nope_dim + c.qk_rope_dim
                if c.q_lora_rank:
                    s.update({p + "attn_q_a": (c.q_lora_rank, H), p + "attn_q_a_norm": (c.q_lora_rank,),
                              p + "attn_q_b": (c.n_heads * qk, c.q_lora_rank)})
                else:
                    s[p + "attn_q"] = (c.n_heads * qk, H)
                s.update({p + "attn_kv_a": (c.kv_lora_rank + c.qk_rope_dim, H), p + "attn_kv_a_norm": (c.kv_lora_rank,),
                          p + "attn_kv_b": (c.n_heads * (c.qk_nope_dim + c.v_head_dim), c.kv_lora_rank),
                          p + "attn_o": (H, c.n_heads * c.v_head_dim)})
                if c.index_topk:
                    s.update({p + "idx_q": (c.index_n_heads * c.index_head_dim, c.q_lora_rank), p + "idx_k": (c.index_head_dim, H),
                              p + "idx_k_norm": (c.index_head_dim,), p + "idx_k_norm_bias": (c.index_head_dim,),
                              p + "idx_weights": (c.index_n_heads, H)})
            elif kind == "attention":
                s.update({p + "attn_q": (c.q_size, H), p + "attn_k": (c.kv_size, H), p + "attn_v": (c.kv_size, H),
                          p + "attn_o": (H, c.q_size)})
                if c.attn_gate:
                    s[p + "attn_gate"] = (c.q_size, H)
                if c.attn_bias:
                    s.update({p + "attn_q_bias": (c.q_size,), p + "attn_k_bias": (c.kv_size,), p + "attn_v_bias": (c.kv_size,)})
                if c.out_bias:
                    s[p + "attn_o_bias"] = (H,)
                if c.qk_norm:
                    s.update({p + "attn_q_norm": (c.q_size if c.qk_norm_wide else D,),
                              p + "attn_k_norm": (c.kv_size if c.qk_norm_wide else D,)})
                if c.attn_sinks:
                    s[p + "attn_sinks"] = (c.n_heads,)
                if c.index_ratio:
                    s.update({p + "idx_q": (c.index_n_heads * c.index_head_dim, H), p + "idx_k": (c.index_head_dim, H),
                              p + "idx_q_norm": (c.index_head_dim,), p + "idx_k_norm": (c.index_head_dim,)})
            if not has_ffn:
                continue
            if c.moe_layer(l):
                s[p + "ffn_router"] = (c.n_experts, H)
                if c.router_bias:
                    s[p + "ffn_router_bias"] = (c.n_experts,)
                if c.router_select_bias:
                    s[p + "ffn_router_select_bias"] = (c.n_experts,)
                s[p + "experts_in"] = (c.n_experts, (2 if c.gated_ffn else 1) * c.moe_ffn, H)      # gate rows then up rows
                s[p + "experts_out"] = (c.n_experts, H, c.moe_ffn)
                if c.expert_bias:
                    s[p + "experts_in_bias"] = (c.n_experts, (2 if c.gated_ffn else 1) * c.moe_ffn)
                    s[p + "experts_out_bias"] = (c.n_experts, H)
                if c.shared_width:
                    Fs = c.shared_width
                    s.update({p + "shared_up": (Fs, H), p + "shared_down": (H, Fs)})
                    if c.gated_ffn:
                        s[p + "shared_gate"] = (Fs, H)
                    if c.shared_expert_gate:
                        s[p + "shared_expert_gate"] = (1, H)
            else:
                if c.gated_ffn:
                    s[p + "ffn_gate"] = (c.ffn, H)
                s.update({p + "ffn_up": (c.ffn, H), p + "ffn_down": (H, c.ffn)})
                if c.mlp_bias:
                    if c.gated_ffn:
                        s[p + "ffn_gate_bias"] = (c.ffn,)
                    s.update({p + "ffn_up_bias": (c.ffn,), p + "ffn_down_bias": (H,)})
        if c.norm_kind == "layer" and c.norm_bias:
            for n in norms:
                s[n + "_bias"] = s[n]
        return s

    # ------------------------------------------------------------------------------------------------------------
    def trace(self, spec: StepSpec) -> Graph:
        c = self.cfg
        b = Builder()
        R, T, cap = spec.rows, spec.tokens, spec.capacity
        H, D, Hq, Hkv = c.hidden, c.head_dim, c.n_heads, c.n_kv_heads
        w = spec.world
        hq, hkv = Hq // w, max(Hkv // w, 1)
        shapes = self.weight_shapes()

        consts: Dict[str, Traced] = {}
        packed_as = dict(spec.weight_formats)

        def W(name: str, shape=None) -> Traced:
            if name not in consts:
                shp = tuple(shape or shapes[name])
                if name in packed_as and len(shp) == 2:
                    from ..quant.formats import packed_nbytes
                    raw = b.const(name, (packed_nbytes(packed_as[name], shp[0] * shp[1]),), DType.U8)
                    consts[name] = b.packed_dequant(raw, packed_as[name], shp)
                else:
                    consts[name] = b.const(name, shp, spec.weight_dtype).cast(F32)
            return consts[name]

        def norm(x: Traced, name: str) -> Traced:
            if c.norm_kind == "layer":
                return O.layernorm(b, x, W(name), W(name + "_bias") if c.norm_bias else None, c.norm_eps)
            return O.rmsnorm(b, x, W(name), c.norm_eps)

        tokens = b.slot("tokens", (R, T), I32, "token", range=(0, c.vocab - 1))
        positions = b.slot("positions", (R, T), I32, "pos", range=(0, c.max_position - 1))
        if spec.paged:
            read_map = b.slot("read_map", (R, cap), I32, "slot_map", range=(0, spec.slots - 1))
            write_map = b.slot("write_map", (R * T,), I32, "write_map", range=(-1, spec.slots - 1))
        rot = c.qk_rope_dim if c.is_mla else c.rot
        rope_tables: Dict[tuple, tuple] = {}
        flat = []

        def rope_of(layer: int):
            """cos / sin rows of this step's positions for the layer's rope base (windowed layers may use their own)."""
            local = c.rope_theta_local is not None and c.window_of(layer) > 0
            key = ("local",) if local else ("global",)
            if key not in rope_tables:
                theta, scaling = (c.rope_theta_local, type(c.rope_scaling)()) if local else (c.rope_theta, c.rope_scaling)
                tag = "rope.local" if local else "rope"
                ct = b.computed(tag + ".cos", (c.max_position, rot), F32, "rope_cos", (rot, theta, c.max_position, scaling))
                st = b.computed(tag + ".sin", (c.max_position, rot), F32, "rope_sin", (rot, theta, c.max_position, scaling))
                rope_tables.setdefault(("table",), (ct, st))
                if not flat:
                    flat.append(b.reshape(positions, (R * T,)))
                if spec.mrope and c.mrope_sections:
                    # sectioned rotary: channel pairs [0, s0) turn with the time stream, [s0, s0 + s1) with the row
                    # stream, the rest with the column stream (multimodal/mrope.rs); text tokens carry three equal values
                    streams = b.slot("rope_positions", (3, R * T), I32, "pos", range=(0, c.max_position - 1))
                    per = [(b.gather(ct, b.reshape(b.slice(streams, 0, i, 1), (R * T,)), 0),
                            b.gather(st, b.reshape(b.slice(streams, 0, i, 1), (R * T,)), 0)) for i in range(3)]
                    half, cuts, at = rot // 2, [], 0
                    for i, n in enumerate(c.mrope_sections):
                        cuts.append((i % 3, at, n))
                        at += n
                    if at != half:
                        raise ValueError(f"mrope sections {c.mrope_sections} do not cover {half} channel pairs")
                    pieces = lambda k: [b.slice(per[i][k], -1, base + a0, n) for base in (0, half) for i, a0, n in cuts]
                    rope_tables[key] = (b.concat(pieces(0), -1), b.concat(pieces(1), -1))
                else:
                    rope_tables[key] = (b.gather(ct, flat[0], 0), b.gather(st, flat[0], 0))
            return rope_tables[key]

        if c.pos == "rope" and c.mixer_of(0) == "attention":
            rope_of(0)
        masks: Dict[int, Traced] = {}

        def mask_of(layer: int) -> Traced:
            win = c.window_of(layer)
            if win not in masks:
                masks[win] = O.causal_mask_from_pos(b, positions, cap, win)
            return masks[win]

        mask_of(0)
        head_bias = None
        if c.pos == "alibi":
            sl = O.alibi_slopes(Hq, c.alibi_slopes, c.alibi_bias_max)
            head_bias = O.alibi_bias_from_pos(b, positions, cap, sl[spec_rank_heads(spec, hq)])

        h = b.gather(W("embed"), b.reshape(tokens, (R * T,)), 0)          # [R*T, H]
        if c.embed_scale != 1.0:
            h = h * c.embed_scale
        if spec.embeds:
            # rows computed outside the text stack (a vision connector's output) stand in for flagged tokens' embeddings
            rows_in = b.slot("embed_rows", (R * T, H), F32, "activation")
            flagged = b.slot("embed_flags", (R * T,), I32, "activation", range=(0, 1))
            h = b.select(b.broadcast(b.reshape(flagged, (R * T, 1)), (R * T, H)), rows_in, h)
        if c.embed_norm:
            h = norm(h, "embed_norm")
        if c.mtp_head:
            # multi-token-prediction input: the embedding of the token that FOLLOWS a position (zeroed at absolute
            # position 0) and the target's closing hidden state of that position, each under its own norm, embedding
            # first, mapped back to the width (DeepSeek-V3 section 2.2; crates/poot-models/src/architectures/
            # glm53_flash/mtp.rs:9-13)
            carry = b.slot("carry", (R * T, H), F32, "activation")
            first = b.binary("ge", b.broadcast(b.scalar(0, I32), (R * T, 1)), b.reshape(positions, (R * T, 1)))   # pos == 0
            h = b.select(b.broadcast(first, (R * T, H)), b.broadcast(b.scalar(0.0, F32), (R * T, H)), h)
            h = O.linear(b, b.concat([norm(h, "mtp.enorm"), norm(carry, "mtp.hnorm")], -1), W("mtp.eh_proj"))
        scale = c.attn_scale if c.attn_scale is not None else 1.0 / math.sqrt(D)
        rs = c.residual_scale

        def kv_through_cache(p: str, k: Traced, v: Traced, dk: int, dv: int):
            """Write this step's keys / values and read the visible window back (through the storage dtype, which keeps
            decode-by-steps equal to one-shot prefill)."""
            nk = k.shape[1]
            if spec.paged:
                kp = b.state(p + "k_pool", (spec.slots, nk, dk), spec.kv_dtype, "blocked").cast(F32)
                vp = b.state(p + "v_pool", (spec.slots, nk, dv), spec.kv_dtype, "blocked").cast(F32)
                kp2 = b.scatter_update(kp, write_map, k)
                vp2 = b.scatter_update(vp, write_map, v)
                b.output(kp2.cast(spec.kv_dtype), p + "k_pool.next", "state_next", p + "k_pool")
                b.output(vp2.cast(spec.kv_dtype), p + "v_pool.next", "state_next", p + "v_pool")
                return (O.paged_view(b, kp2.cast(spec.kv_dtype).cast(F32), read_map),
                        O.paged_view(b, vp2.cast(spec.kv_dtype).cast(F32), read_map))
            kc = b.state(p + "k_cache", (R, nk, cap, dk), spec.kv_dtype, "positional", 2).cast(F32)
            vc = b.state(p + "v_cache", (R, nk, cap, dv), spec.kv_dtype, "positional", 2).cast(F32)
            start = b.slice(b.reshape(positions, (R * T,)), 0, 0, 1)
            kn = b.transpose(b.reshape(k, (R, T, nk, dk)), (0, 2, 1, 3))
            vn = b.transpose(b.reshape(v, (R, T, nk, dv)), (0, 2, 1, 3))
            kc2 = b.dynamic_update_slice(kc, kn, start, 2)
            vc2 = b.dynamic_update_slice(vc, vn, start, 2)
            b.output(kc2.cast(spec.kv_dtype), p + "k_cache.next", "state_next", p + "k_cache")
            b.output(vc2.cast(spec.kv_dtype), p + "v_cache.next", "state_next", p + "v_cache")
            return kc2.cast(spec.kv_dtype).cast(F32), vc2.cast(spec.kv_dtype).cast(F32)

        def attention(l: int, x: Traced) -> Traced:
            p = f"layers.{l}."
            if c.is_mla:
                return mla_attention(l, x)
            bias = (lambda n, k_: W(p + n, (k_,))) if c.attn_bias else (lambda n, k_: None)
            q = O.linear(b, x, W(p + "attn_q", (hq * D, H)), bias("attn_q_bias", hq * D))
            k = O.linear(b, x, W(p + "attn_k", (hkv * D, H)), bias("attn_k_bias", hkv * D))
            v = O.linear(b, x, W(p + "attn_v", (hkv * D, H)), bias("attn_v_bias", hkv * D))
            if c.qk_norm and c.qk_norm_wide:
                q = O.rmsnorm(b, q, W(p + "attn_q_norm"), c.norm_eps)
                k = O.rmsnorm(b, k, W(p + "attn_k_norm"), c.norm_eps)
            q = b.reshape(q, (R * T, hq, D))
            k = b.reshape(k, (R * T, hkv, D))
            v = b.reshape(v, (R * T, hkv, D))
            if c.qk_norm and not c.qk_norm_wide:
                q = O.rmsnorm(b, q, W(p + "attn_q_norm"), c.norm_eps)
                k = O.rmsnorm(b, k, W(p + "attn_k_norm"), c.norm_eps)
            if c.uses_rope(l):
                cos, sin = rope_of(l)
                q = O.rope(b, q, cos, sin, rot)
                k = O.rope(b, k, cos, sin, rot)
            K, V = kv_through_cache(p, k, v, D, D)
            qh = b.transpose(b.reshape(q, (R, T, hq, D)), (0, 2, 1, 3))
            a = O.attention_biased(b, qh, K, V, block_mask(l, x) if c.index_ratio else mask_of(l), scale, hq // hkv, c.attn_softcap, head_bias,
                                   W(p + "attn_sinks", (hq,)) if c.attn_sinks else None)
            a = b.reshape(b.transpose(a, (0, 2, 1, 3)), (R * T, hq * D))
            if c.attn_gate:
                a = a * O.sigmoid(b, O.linear(b, x, W(p + "attn_gate", (hq * D, H))))
            o = O.linear(b, a, W(p + "attn_o", (H, hq * D)))
            if w > 1:
                o = b.all_reduce(o)
            if c.out_bias:
                o = o + b.broadcast(W(p + "attn_o_bias"), o.shape)
            return o

        def block_mask(l: int, x: Traced) -> Traced:
            """Block indexer (architectures/qwen38/qsa.rs): per-head queries (RMSNorm, partial rotary at the token's
            position) score BLOCKS of ``index_ratio`` positions, ``sum_h relu(q_h . k_b) / sqrt(dim)``; a block's key is
            the mean of its positions' raw keys, then RMSNorm, then rotary at the block's first position.  A block is
            eligible once all of it is at or before the query; the ``index_budget // index_ratio`` best stay (equal
            scores: the lower block) with all their positions.  The query's own unfinished block is always read,
            unscored; a query on the last position of its block reads that block only if it is selected.  The raw keys
            are cached per position (``idx_pool``) and the block keys recomputed from them."""
            if not spec.paged or cap % c.index_ratio or c.window_of(l):
                raise ValueError("the block indexer is traced over paged pools whose capacity is a whole number of blocks, without a window")
            p = f"layers.{l}."
            ni, di, ratio = c.index_n_heads, c.index_head_dim, c.index_ratio
            nb = cap // ratio
            cos, sin = rope_of(l)
            q = O.rope(b, O.rmsnorm(b, b.reshape(O.linear(b, x, W(p + "idx_q")), (R * T, ni, di)), W(p + "idx_q_norm"), c.norm_eps), cos, sin, rot)
            pool = b.state(p + "idx_pool", (spec.slots, 1, di), spec.kv_dtype, "blocked").cast(F32)
            pool2 = b.scatter_update(pool, write_map, b.reshape(O.linear(b, x, W(p + "idx_k")), (R * T, 1, di)))
            b.output(pool2.cast(spec.kv_dtype), p + "idx_pool.next", "state_next", p + "idx_pool")
            raw = O.paged_view(b, pool2.cast(spec.kv_dtype).cast(F32), read_map)                      # [R, 1, cap, di]
            pooled = b.reshape(raw, (R, nb, ratio, di)).sum(2) * (1.0 / ratio)
            key = (c.rope_theta, "blocks", ratio, nb)
            if key not in rope_tables:
                ct, st = rope_tables[("table",)]
                starts = b.iota((nb,), 0) * ratio
                rope_tables[key] = tuple(b.reshape(b.broadcast(b.reshape(b.gather(t_, starts, 0), (1, nb, rot)), (R, nb, rot)), (R * nb, rot))
                                         for t_ in (ct, st))
            bc, bs = rope_tables[key]
            kb = O.rope(b, b.reshape(O.rmsnorm(b, pooled, W(p + "idx_k_norm"), c.norm_eps), (R * nb, 1, di)), bc, bs, rot)
            qh = b.transpose(b.reshape(q, (R, T, ni, di)), (0, 2, 1, 3))
            kt = b.broadcast(b.reshape(b.transpose(b.reshape(kb, (R, nb, di)), (0, 2, 1)), (R, 1, di, nb)), (R, ni, di, nb))
            score = O.relu(b, b.matmul(qh, kt, "exact")).sum(1) * (di ** -0.5)                        # [R, T, nb]
            pos3 = lambda n: b.broadcast(b.reshape(positions, (R, T, 1)), (R, T, n))
            eligible = b.binary("ge", pos3(nb), b.iota((R, T, nb), 2) * ratio + (ratio - 1))
            score = b.select(eligible, O.canonical_router_scores(b, score), b.broadcast(b.scalar(-O.F32_MAX, F32), score.shape))
            kept = min(c.index_budget // ratio, nb)
            rank = b.reshape(O.stable_descending_rank(b, b.reshape(score, (R * T, nb))), (R, T, nb))
            chosen = b.binary("and", O.lnot(b, b.binary("ge", rank, b.broadcast(b.scalar(kept, I32), rank.shape))), eligible)
            spread = b.reshape(b.broadcast(b.reshape(chosen, (R, T, nb, 1)), (R, T, nb, ratio)), (R, T, cap))
            slots_ = b.iota((R, T, cap), 2)
            own_from = b.cast(eligible, I32).sum(-1, keepdim=True) * ratio                           # first position past the complete blocks
            own = b.binary("and", b.binary("ge", slots_, b.broadcast(own_from, (R, T, cap))), b.binary("ge", pos3(cap), slots_))
            keep = b.binary("or", spread, own)
            return b.select(keep, b.broadcast(b.scalar(0.0, F32), (R, T, cap)), b.broadcast(b.scalar(O.MASK_HIDDEN, F32), (R, T, cap)))

        def sparse_mask(p: str, x: Traced, q_resid: Traced, cos: Traced, sin: Traced, mask: Traced) -> Traced:
            """Sparse attention indexer (components/dsa.rs): a light multi-head scorer over its own cached keys ranks the
            visible keys of every query, ``score[t, s] = sum_h w[t, h] * relu(q[t, h] . k[s]) / sqrt(Di)``; the
            ``index_topk`` best stay visible to the main attention.  The rotary part leads each indexer head and is
            rotated half-split."""
            ni, Di, dr = c.index_n_heads, c.index_head_dim, c.qk_rope_dim
            q = b.reshape(O.linear(b, q_resid, W(p + "idx_q")), (R * T, ni, Di))
            q = b.concat([O.rope(b, b.slice(q, -1, 0, dr), cos, sin, dr), b.slice(q, -1, dr, Di - dr)], -1)
            k = O.layernorm(b, O.linear(b, x, W(p + "idx_k")), W(p + "idx_k_norm"), W(p + "idx_k_norm_bias"), 1e-6)
            k = b.reshape(k, (R * T, 1, Di))
            k = b.concat([O.rope(b, b.slice(k, -1, 0, dr), cos, sin, dr), b.slice(k, -1, dr, Di - dr)], -1)
            if not spec.paged:
                raise ValueError("the sparse attention indexer is traced over paged pools")
            pool = b.state(p + "idx_pool", (spec.slots, 1, Di), spec.kv_dtype, "blocked").cast(F32)
            pool2 = b.scatter_update(pool, write_map, k)
            b.output(pool2.cast(spec.kv_dtype), p + "idx_pool.next", "state_next", p + "idx_pool")
            keys = O.paged_view(b, pool2.cast(spec.kv_dtype).cast(F32), read_map)            # [R, 1, cap, Di]
            qh = b.transpose(b.reshape(q, (R, T, ni, Di)), (0, 2, 1, 3))                        # [R, ni, T, Di]
            kt = b.broadcast(b.transpose(keys, (0, 1, 3, 2)), (R, ni, Di, cap))
            dots = O.relu(b, b.matmul(qh, kt, "exact") * (Di ** -0.5))                          # [R, ni, T, cap]
            wts = O.linear(b, x, W(p + "idx_weights"), precision="exact") * (ni ** -0.5)        # [R*T, ni]
            wts = b.transpose(b.reshape(wts, (R, T, ni)), (0, 2, 1))
            score = (dots * b.broadcast(b.reshape(wts, (R, ni, T, 1)), dots.shape)).transpose(0, 2, 3, 1).sum(-1) + mask
            rank = b.reshape(O.stable_descending_rank(b, b.reshape(score, (R * T, cap))), (R, T, cap))
            keep = O.lnot(b, b.binary("ge", rank, b.broadcast(b.scalar(c.index_topk, I32), rank.shape)))
            return b.select(keep, mask, b.broadcast(b.scalar(O.MASK_HIDDEN, F32), mask.shape))

        def mla_attention(l: int, x: Traced) -> Traced:
            """Multi-head latent attention in its expanded (prefill) form: queries and keys are the concatenation of a
            per-head no-position part and a rotary part; the rotary key is one head shared by all (components/mla.rs)."""
            p = f"layers.{l}."
            dn, dr, dv, nh = c.qk_nope_dim, c.qk_rope_dim, c.v_head_dim, c.n_heads
            if c.q_lora_rank:
                qa = O.rmsnorm(b, O.linear(b, x, W(p + "attn_q_a")), W(p + "attn_q_a_norm"), c.mla_eps)
                q = O.linear(b, qa, W(p + "attn_q_b"))
            else:
                qa = None
                q = O.linear(b, x, W(p + "attn_q"))
            q = b.reshape(q, (R * T, nh, dn + dr))
            kva = O.linear(b, x, W(p + "attn_kv_a"))                          # [L, kv_lora + dr]
            ckv = O.rmsnorm(b, b.slice(kva, -1, 0, c.kv_lora_rank), W(p + "attn_kv_a_norm"), c.mla_eps)
            k_rope = b.reshape(b.slice(kva, -1, c.kv_lora_rank, dr), (R * T, 1, dr))
            kvb = b.reshape(O.linear(b, ckv, W(p + "attn_kv_b")), (R * T, nh, dn + dv))
            cos, sin = rope_of(l)
            q_rope = O.rope(b, b.slice(q, -1, dn, dr), cos, sin, dr)
            k_rope = O.rope(b, k_rope, cos, sin, dr)
            qf = b.concat([b.slice(q, -1, 0, dn), q_rope], -1)
            kf = b.concat([b.slice(kvb, -1, 0, dn), b.broadcast(k_rope, (R * T, nh, dr))], -1)
            vf = b.slice(kvb, -1, dn, dv)
            K, V = kv_through_cache(p, kf, vf, dn + dr, dv)
            qh = b.transpose(b.reshape(qf, (R, T, nh, dn + dr)), (0, 2, 1, 3))
            mask = mask_of(l)
            if c.index_topk:
                mask = sparse_mask(p, x, qa, cos, sin, mask)
            a = O.attention_masked(b, qh, K, V, mask, scale, 1, 0.0)
            a = b.reshape(b.transpose(a, (0, 2, 1, 3)), (R * T, nh * dv))
            return O.linear(b, a, W(p + "attn_o"))

        def dense_ffn(x: Traced, p: str, gate: str, up: str, down: str, F: int) -> Traced:
            mb = (lambda n, k_: W(p + n, (k_,))) if c.mlp_bias else (lambda n, k_: None)
            if c.gated_ffn:
                g_ = O.linear(b, x, W(p + gate, (F, H)), mb(gate + "_bias", F))
                u_ = O.linear(b, x, W(p + up, (F, H)), mb(up + "_bias", F))
                a = O.swiglu(b, g_, u_) if c.act == "silu" else O.ffn_activation(b, g_, u_, c.act)
            else:
                a = O.ffn_activation(b, O.linear(b, x, W(p + up, (F, H)), mb(up + "_bias", F)), None, c.act)
            f = O.linear(b, a, W(p + down, (H, F)))
            if w > 1:
                f = b.all_reduce(f)
            if c.mlp_bias:
                f = f + b.broadcast(W(p + down + "_bias"), f.shape)
            return f

        def ffn(l: int, x: Traced) -> Traced:
            p = f"layers.{l}."
            if not c.moe_layer(l):
                return dense_ffn(x, p, "ffn_gate", "ffn_up", "ffn_down", c.ffn // w)
            plain = (c.router == "softmax" and c.norm_topk_prob and not (c.router_bias or c.router_select_bias or c.expert_bias)
                     and c.n_group == 1 and c.routed_scale == 1.0 and c.act == "silu" and c.swiglu_limit == 0 and c.gated_ffn)
            if plain:
                f = O.moe_topk_softmax(b, x, W(p + "ffn_router"), W(p + "experts_in"), W(p + "experts_out"), c.top_k)
            else:
                f = O.moe_routed(
                    b, x, W(p + "ffn_router"), W(p + "experts_in"), W(p + "experts_out"), c.top_k, score=c.router,
                    renorm=c.norm_topk_prob, router_bias=W(p + "ffn_router_bias") if c.router_bias else None,
                    select_bias=W(p + "ffn_router_select_bias") if c.router_select_bias else None, n_group=c.n_group,
                    topk_group=c.topk_group, routed_scale=c.routed_scale, act=c.act, limit=c.swiglu_limit,
                    alpha=c.swiglu_alpha, in_bias=W(p + "experts_in_bias") if c.expert_bias else None,
                    out_bias=W(p + "experts_out_bias") if c.expert_bias else None, gated=c.gated_ffn)
            if c.shared_width:
                sh = dense_ffn(x, p, "shared_gate", "shared_up", "shared_down", c.shared_width)
                if c.shared_expert_gate:
                    sh = sh * b.broadcast(O.sigmoid(b, O.linear(b, x, W(p + "shared_expert_gate"))), sh.shape)
                f = f + sh
            return f

        def recurrent_state(name: str, shape):
            st = b.state(name, shape, F32, "recurrent")
            return st

        def mamba(l: int, x: Traced) -> Traced:
            """Mamba2 mixer (components/mamba2.rs): in-projection -> causal depthwise conv + SiLU over (x | B | C) ->
            selective state-space scan per head -> gated grouped RMSNorm -> out-projection."""
            p = f"layers.{l}."
            nh, P, N, G, K = c.ssm_heads, c.ssm_head_dim, c.ssm_state, c.ssm_groups, c.ssm_conv
            I = nh * P
            C = I + 2 * G * N
            z = O.linear(b, x, W(p + "ssm_in_z"))
            xbc = O.linear(b, x, W(p + "ssm_in_x"))
            dt = O.softplus_stable(b, O.linear(b, x, W(p + "ssm_in_dt")) + b.broadcast(W(p + "ssm_dt_bias"), (R * T, nh)))
            conv_in = recurrent_state(p + "conv_state", (R, K - 1, C))
            ssm_in = recurrent_state(p + "ssm_state", (R, nh, N, P))
            a = b.reshape(-b.unary("exp", W(p + "ssm_a_log")), (1, nh, 1, 1))
            d = b.reshape(W(p + "ssm_d"), (1, nh, 1, 1))
            ys, convs, states = [], [], []
            for r in range(R):
                xr = b.slice(xbc, 0, r * T, T)
                y, cs = O.causal_conv1d(b, xr, b.reshape(b.slice(conv_in, 0, r, 1), (K - 1, C)), W(p + "ssm_conv"),
                                        W(p + "ssm_conv_bias") if c.ssm_conv_bias else None)
                y = O.silu(b, y)
                xs = b.transpose(b.reshape(b.slice(y, 1, 0, I), (1, T, nh, P)), (0, 2, 1, 3))            # [1, nh, T, P]
                group = lambda t: O.repeat_kv(b, b.transpose(b.reshape(t, (1, T, G, N)), (0, 2, 1, 3)), nh // G)
                Bm, Cm = group(b.slice(y, 1, I, G * N)), group(b.slice(y, 1, I + G * N, G * N))
                dtr = b.reshape(b.transpose(b.slice(dt, 0, r * T, T), (1, 0)), (1, nh, T, 1))
                yo, so = b.scan("ssd", [xs, Bm, Cm, dtr, a, d, b.slice(ssm_in, 0, r, 1)])
                ys.append(b.reshape(b.transpose(yo, (0, 2, 1, 3)), (T, I)))
                convs.append(b.reshape(cs, (1, K - 1, C)))
                states.append(so)
            b.output(b.concat(convs, 0) if R > 1 else convs[0], p + "conv_state.next", "state_next", p + "conv_state")
            b.output(b.concat(states, 0) if R > 1 else states[0], p + "ssm_state.next", "state_next", p + "ssm_state")
            y = b.concat(ys, 0) if R > 1 else ys[0]
            # gate, then RMSNorm within each of the G channel groups
            gated = y * O.silu(b, z)
            gn = O.rmsnorm(b, b.reshape(gated, (R * T, G, I // G)), b.reshape(W(p + "ssm_gate_norm_w"), (G, I // G)), c.norm_eps)
            return O.linear(b, b.reshape(gn, (R * T, I)), W(p + "ssm_o"))

        def gdn(l: int, x: Traced) -> Traced:
            """Gated delta net mixer (components/gdn.rs): projections -> causal conv + SiLU over (q | k | v) -> unit-norm
            q and k -> gated delta rule scan per value head -> RMSNorm gated by SiLU(z) -> out-projection."""
            p = f"layers.{l}."
            nk, nv, Dg, K = c.gdn_k_heads, c.gdn_v_heads, c.gdn_head_dim, c.gdn_conv
            C = (2 * nk + nv) * Dg
            mixed = b.concat([O.linear(b, x, W(p + "gdn_q")), O.linear(b, x, W(p + "gdn_k")), O.linear(b, x, W(p + "gdn_v"))], -1)
            z = b.reshape(O.linear(b, x, W(p + "gdn_z")), (R * T, nv, Dg))
            beta = O.sigmoid(b, O.linear(b, x, W(p + "gdn_b")))                                             # [L, nv]
            sp = O.softplus_stable(b, O.linear(b, x, W(p + "gdn_a")) + b.broadcast(W(p + "gdn_dt_bias"), (R * T, nv)))
            g = -(b.broadcast(b.unary("exp", W(p + "gdn_a_log")), (R * T, nv)) * sp)
            conv_in = recurrent_state(p + "conv_state", (R, K - 1, C))
            s_in = recurrent_state(p + "gdn_state", (R, nv, Dg, Dg))
            ys, convs, states = [], [], []
            for r in range(R):
                y, cs = O.causal_conv1d(b, b.slice(mixed, 0, r * T, T), b.reshape(b.slice(conv_in, 0, r, 1), (K - 1, C)),
                                        W(p + "gdn_conv"))
                y = O.silu(b, y)
                heads = lambda t, n: b.transpose(b.reshape(t, (1, T, n, Dg)), (0, 2, 1, 3))
                q = O.repeat_kv(b, O.l2norm(b, heads(b.slice(y, 1, 0, nk * Dg), nk)), nv // nk) * (1.0 / math.sqrt(Dg))
                k = O.repeat_kv(b, O.l2norm(b, heads(b.slice(y, 1, nk * Dg, nk * Dg), nk)), nv // nk)
                v = heads(b.slice(y, 1, 2 * nk * Dg, nv * Dg), nv)
                col = lambda t: b.reshape(b.transpose(b.slice(t, 0, r * T, T), (1, 0)), (1, nv, T, 1))
                if spec.gdn_chunk > 0 and T > 1:
                    yo, so = O.delta_rule_chunked(b, q, k, v, col(g), col(beta), b.slice(s_in, 0, r, 1), spec.gdn_chunk)
                else:
                    yo, so = b.scan("delta_rule", [q, k, v, col(g), col(beta), b.slice(s_in, 0, r, 1)])
                ys.append(b.reshape(b.transpose(yo, (0, 2, 1, 3)), (T, nv, Dg)))
                convs.append(b.reshape(cs, (1, K - 1, C)))
                states.append(so)
            b.output(b.concat(convs, 0) if R > 1 else convs[0], p + "conv_state.next", "state_next", p + "conv_state")
            b.output(b.concat(states, 0) if R > 1 else states[0], p + "gdn_state.next", "state_next", p + "gdn_state")
            y = b.concat(ys, 0) if R > 1 else ys[0]
            out = O.gated_rmsnorm(b, y, z, W(p + "gdn_gate_norm_w"), c.norm_eps, gate_first=False, gate_act=c.gdn_gate_act)
            return O.linear(b, b.reshape(out, (R * T, nv * Dg)), W(p + "gdn_o"))

        mixers = {"attention": attention, "mamba": mamba, "gdn": gdn}
        S, L = c.hc_count, R * T

        def grouped_norm(x: Traced, name: str) -> Traced:
            """RMSNorm of each of the ``S`` runs of ``H`` values of ``x[L, S * H]`` by its own mean square, then one scale
            over the whole row (components/ple.rs ``grouped_norm``)."""
            g3 = b.reshape(x, (L, S, H))
            den = b.unary("sqrt", (g3 * g3).sum(-1, keepdim=True) * (1.0 / H) + c.norm_eps)
            return b.reshape(g3 / b.broadcast(den, g3.shape), (L, S * H)) * b.broadcast(W(name), (L, S * H))

        def hc_read(xs: Traced, stem: str, inject: bool):
            """A gate of the hyper-connections (architectures/qwen38/gated_residual.rs): the block's input is the mean
            over the streams of ``sigmoid(up(silu(down(n) / S))) * n`` with ``n`` the grouped norm of the streams; the
            weights that write the block's output back are ``2 * sigmoid(inject(n) / S)`` per stream."""
            n = grouped_norm(xs, stem + "norm")
            gate = O.sigmoid(b, O.linear(b, O.silu(b, O.linear(b, n, W(stem + "down")) * (1.0 / S)), W(stem + "up")))
            x_in = b.reshape(gate * n, (L, S, H)).sum(1) * (1.0 / S)
            return x_in, (O.sigmoid(b, O.linear(b, n, W(stem + "inject")) * (1.0 / S)) * 2.0 if inject else None)

        def hc_write(xs: Traced, out: Traced, weights: Traced) -> Traced:
            placed = b.broadcast(b.reshape(out, (L, 1, H)), (L, S, H)) * b.broadcast(b.reshape(weights, (L, S, 1)), (L, S, H))
            return xs + b.reshape(placed, (L, S * H))

        def ple(l: int, xs: Traced) -> Traced:
            """Per-layer embedding block (components/ple.rs): hashed n-gram ids of the step's tokens (the ``ngram_size -
            1`` tokens before the step are carried per sequence, xor-ed with the end-of-sequence id so that a zero
            state reads as a sequence start) look up one table row per hash head; the rows' key, under a grouped norm,
            gates their value into every stream by its agreement with the normed streams,
            ``sigmoid(sign(g) * sqrt(max(|g|, 1e-6)))`` with ``g = key . query / sqrt(H)``; a dilated depthwise causal conv
            of the normed result, through SiLU, is added to it."""
            p = f"layers.{l}."
            tb = c.ple_tables(l)
            ctx, heads, dil, K = c.ngram_size - 1, len(tb.primes), c.ngram_size, c.ple_conv
            hist = b.state(p + "ple_history", (R, ctx), I32, "recurrent")
            eos = b.broadcast(b.scalar(c.eos_token, I32), (ctx,))
            ids, nxt = [], []
            for r in range(R):
                win = b.concat([b.binary("xor", b.reshape(b.slice(hist, 0, r, 1), (ctx,)), eos), b.reshape(b.slice(tokens, 0, r, 1), (T,))], 0)
                ids.append(b.ngram_hash(win, ctx, tb.multipliers, tb.primes, tb.offsets, c.heads_per_ngram, c.eos_token))
                nxt.append(b.reshape(b.binary("xor", b.slice(win, 0, T, ctx), eos), (1, ctx)))
            b.output(b.concat(nxt, 0) if R > 1 else nxt[0], p + "ple_history.next", "state_next", p + "ple_history")
            ids = b.concat(ids, 0) if R > 1 else ids[0]                                           # [L, heads]
            emb = b.reshape(b.gather(W(p + "ple_table"), b.reshape(ids, (L * heads,)), 0), (L, c.ple_embed_dim))
            key = grouped_norm(O.linear(b, emb, W(p + "ple_key")), p + "ple_key_norm")
            value = O.linear(b, emb, W(p + "ple_value"))
            query = grouped_norm(xs, p + "ple_query_norm")
            g_ = b.reshape(key * query, (L, S, H)).sum(-1, keepdim=True) * (H ** -0.5)           # [L, S, 1]
            mag = b.unary("sqrt", b.binary("max", b.binary("max", g_, -g_), b.broadcast(b.scalar(1e-6, F32), g_.shape)))
            zero = b.broadcast(b.scalar(0.0, F32), g_.shape)
            sign = b.cast(b.binary("ge", g_, zero), F32) - b.cast(b.binary("ge", -g_, zero), F32)
            gated = b.reshape(b.broadcast(O.sigmoid(b, mag * sign), (L, S, H)) * b.broadcast(b.reshape(value, (L, 1, H)), (L, S, H)), (L, S * H))
            n = grouped_norm(gated, p + "ple_conv_norm")
            win_in = b.state(p + "ple_conv_state", (R, (K - 1) * dil, S * H), F32, "recurrent")
            ys, wins = [], []
            for r in range(R):
                y, ws = O.causal_conv1d_dilated(b, b.slice(n, 0, r * T, T), b.reshape(b.slice(win_in, 0, r, 1), ((K - 1) * dil, S * H)),
                                                W(p + "ple_conv"), dil)
                ys.append(y)
                wins.append(b.reshape(ws, (1, (K - 1) * dil, S * H)))
            b.output(b.concat(wins, 0) if R > 1 else wins[0], p + "ple_conv_state.next", "state_next", p + "ple_conv_state")
            return gated + O.silu(b, b.concat(ys, 0) if R > 1 else ys[0])

        if S:
            if c.block != "pre" or c.residual_scale != 1.0:
                raise ValueError("gated hyper-connections are traced for plain pre-gate blocks")
            xs = b.reshape(b.broadcast(b.reshape(h, (L, 1, H)), (L, S, H)), (L, S * H))
            for l in range(c.n_layers):
                p = f"layers.{l}."
                if c.ple_tables(l) is not None:
                    xs = xs + ple(l, xs)                  # reads the raw streams, before the layer's first gate
                x_in, wts = hc_read(xs, p + "hc_attn_", True)
                xs = hc_write(xs, mixers[c.mixer_of(l)](l, x_in), wts)
                x_in, wts = hc_read(xs, p + "hc_ffn_", True)
                xs = hc_write(xs, ffn(l, x_in), wts)
            h = hc_read(xs, "hc_final_", False)[0]        # the closing gate feeds the head directly: no final norm
        for l in range(c.n_layers if not S else 0):
            p = f"layers.{l}."
            kind = c.mixer_of(l)
            if kind != "none":
                o = mixers[kind](l, norm(h, p + "attn_norm") if c.block != "post" else h)
                if c.block != "pre":
                    o = norm(o, p + "attn_post_norm")
                h = h + (o * rs if rs != 1.0 else o)
            if not c.has_ffn(l):
                continue
            f = ffn(l, norm(h, p + "ffn_norm") if c.block != "post" else h)
            if c.block != "pre":
                f = norm(f, p + "ffn_post_norm")
            h = h + (f * rs if rs != 1.0 else f)
        h = b.reshape(h, (R, T, H))
        if spec.logit_rows == "last":
            h = b.reshape(b.slice(h, 1, T - 1, 1), (R, H))
        else:
            h = b.reshape(h, (R * T, H))
        x = h if S else norm(h, "final_norm")
        if spec.carry or c.mtp_head:
            b.output(x, "hidden", "export")
        head = W("embed") if c.tie_embeddings else W("lm_head")
        logits = O.linear(b, x, head)
        if c.logit_scale != 1.0:
            logits = logits * c.logit_scale
        if c.final_softcap > 0:
            logits = O.softcap(b, logits, c.final_softcap)
        if spec.sampler is None:
            b.output(logits, "logits", "result")
        else:
            rows = logits.shape[0]
            seed = params = top_k = None
            if spec.sampler != "greedy":
                seed = b.slot("sampler.seed", (rows,), I32, "owned")
                params = b.slot("sampler.params", (rows, 4 if spec.sampler == "gumbel_top_k_top_p" else 3), F32, "owned")
                if spec.sampler != "gumbel":
                    top_k = b.slot("sampler.top_k", (rows,), I32, "owned")
            b.output(O.sample_head(b, logits, spec.sampler, seed, params, top_k), "picked", "result")
            b.output(logits, "logits", "export")
        return b.finish()
