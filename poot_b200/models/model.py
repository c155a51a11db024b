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

    @property
    def slots(self) -> int:
        return self.pool_slots or self.rows * self.capacity


class Model:
    """One loaded architecture: configuration + tracer + weight-name tables."""

    def __init__(self, cfg: DecoderConfig):
        self.cfg = cfg

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H, D = c.hidden, c.head_dim
        s = {"embed": (c.vocab, H), "final_norm": (H,)}
        if not c.tie_embeddings:
            s["lm_head"] = (c.vocab, H)
        for l in range(c.n_layers):
            p = f"layers.{l}."
            s.update({p + "attn_norm": (H,), p + "attn_q": (c.q_size, H), p + "attn_k": (c.kv_size, H),
                      p + "attn_v": (c.kv_size, H), p + "attn_o": (H, c.q_size), p + "ffn_norm": (H,)})
            if c.attn_bias:
                s.update({p + "attn_q_bias": (c.q_size,), p + "attn_k_bias": (c.kv_size,), p + "attn_v_bias": (c.kv_size,)})
            if c.qk_norm:
                s.update({p + "attn_q_norm": (D,), p + "attn_k_norm": (D,)})
            if c.is_moe:
                s[p + "ffn_router"] = (c.n_experts, H)
                s[p + "experts_in"] = (c.n_experts, 2 * c.moe_ffn, H)      # gate rows then up rows
                s[p + "experts_out"] = (c.n_experts, H, c.moe_ffn)
            else:
                s.update({p + "ffn_gate": (c.ffn, H), p + "ffn_up": (c.ffn, H), p + "ffn_down": (H, c.ffn)})
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

        def W(name: str, shape=None) -> Traced:
            if name not in consts:
                consts[name] = b.const(name, shape or shapes[name], spec.weight_dtype).cast(F32)
            return consts[name]

        tokens = b.slot("tokens", (R, T), I32, "token", range=(0, c.vocab - 1))
        positions = b.slot("positions", (R, T), I32, "pos", range=(0, c.max_position - 1))
        if spec.paged:
            read_map = b.slot("read_map", (R, cap), I32, "slot_map", range=(0, spec.slots - 1))
            write_map = b.slot("write_map", (R * T,), I32, "write_map", range=(-1, spec.slots - 1))
        rot = c.rot
        cos_t = b.computed("rope.cos", (c.max_position, rot), F32, "rope_cos", (rot, c.rope_theta, c.max_position, c.rope_scaling))
        sin_t = b.computed("rope.sin", (c.max_position, rot), F32, "rope_sin", (rot, c.rope_theta, c.max_position, c.rope_scaling))
        flat_pos = b.reshape(positions, (R * T,))
        cos = b.gather(cos_t, flat_pos, 0)
        sin = b.gather(sin_t, flat_pos, 0)
        mask = O.causal_mask_from_pos(b, positions, cap, c.sliding_window)

        h = b.gather(W("embed"), b.reshape(tokens, (R * T,)), 0)          # [R*T, H]
        if c.embed_scale != 1.0:
            h = h * c.embed_scale
        scale = 1.0 / math.sqrt(D)
        for l in range(c.n_layers):
            p = f"layers.{l}."
            x = O.rmsnorm(b, h, W(p + "attn_norm"), c.norm_eps)
            q = O.linear(b, x, W(p + "attn_q", (hq * D, H)), W(p + "attn_q_bias", (hq * D,)) if c.attn_bias else None)
            k = O.linear(b, x, W(p + "attn_k", (hkv * D, H)), W(p + "attn_k_bias", (hkv * D,)) if c.attn_bias else None)
            v = O.linear(b, x, W(p + "attn_v", (hkv * D, H)), W(p + "attn_v_bias", (hkv * D,)) if c.attn_bias else None)
            q = b.reshape(q, (R * T, hq, D))
            k = b.reshape(k, (R * T, hkv, D))
            v = b.reshape(v, (R * T, hkv, D))
            if c.qk_norm:
                q = O.rmsnorm(b, q, W(p + "attn_q_norm"), c.norm_eps)
                k = O.rmsnorm(b, k, W(p + "attn_k_norm"), c.norm_eps)
            q = O.rope(b, q, cos, sin, rot)
            k = O.rope(b, k, cos, sin, rot)
            if spec.paged:
                kp = b.state(p + "k_pool", (spec.slots, hkv, D), spec.kv_dtype, "blocked").cast(F32)
                vp = b.state(p + "v_pool", (spec.slots, hkv, D), spec.kv_dtype, "blocked").cast(F32)
                kp2 = b.scatter_update(kp, write_map, k)
                vp2 = b.scatter_update(vp, write_map, v)
                b.output(kp2.cast(spec.kv_dtype), p + "k_pool.next", "state_next", p + "k_pool")
                b.output(vp2.cast(spec.kv_dtype), p + "v_pool.next", "state_next", p + "v_pool")
                # reading back through the storage dtype keeps decode-by-steps equal to one-shot prefill
                K = O.paged_view(b, kp2.cast(spec.kv_dtype).cast(F32), read_map)
                V = O.paged_view(b, vp2.cast(spec.kv_dtype).cast(F32), read_map)
            else:
                kc = b.state(p + "k_cache", (R, hkv, cap, D), spec.kv_dtype, "positional", 2).cast(F32)
                vc = b.state(p + "v_cache", (R, hkv, cap, D), spec.kv_dtype, "positional", 2).cast(F32)
                start = b.slice(b.reshape(positions, (R * T,)), 0, 0, 1)
                kn = b.transpose(b.reshape(k, (R, T, hkv, D)), (0, 2, 1, 3))
                vn = b.transpose(b.reshape(v, (R, T, hkv, D)), (0, 2, 1, 3))
                kc2 = b.dynamic_update_slice(kc, kn, start, 2)
                vc2 = b.dynamic_update_slice(vc, vn, start, 2)
                b.output(kc2.cast(spec.kv_dtype), p + "k_cache.next", "state_next", p + "k_cache")
                b.output(vc2.cast(spec.kv_dtype), p + "v_cache.next", "state_next", p + "v_cache")
                K, V = kc2.cast(spec.kv_dtype).cast(F32), vc2.cast(spec.kv_dtype).cast(F32)
            qh = b.transpose(b.reshape(q, (R, T, hq, D)), (0, 2, 1, 3))
            a = O.attention_masked(b, qh, K, V, mask, scale, hq // hkv, c.attn_softcap)
            a = b.reshape(b.transpose(a, (0, 2, 1, 3)), (R * T, hq * D))
            o = O.linear(b, a, W(p + "attn_o", (H, hq * D)))
            if w > 1:
                o = b.all_reduce(o)
            h = h + (o * c.residual_scale if c.residual_scale != 1.0 else o)
            x = O.rmsnorm(b, h, W(p + "ffn_norm"), c.norm_eps)
            if c.is_moe:
                f = O.moe_topk_softmax(b, x, W(p + "ffn_router"), W(p + "experts_in"), W(p + "experts_out"), c.top_k)
            else:
                F = c.ffn // w
                g_ = O.linear(b, x, W(p + "ffn_gate", (F, H)))
                u_ = O.linear(b, x, W(p + "ffn_up", (F, H)))
                f = O.linear(b, O.swiglu(b, g_, u_), W(p + "ffn_down", (H, F)))
                if w > 1:
                    f = b.all_reduce(f)
            h = h + (f * c.residual_scale if c.residual_scale != 1.0 else f)
        h = b.reshape(h, (R, T, H))
        if spec.logit_rows == "last":
            h = b.reshape(b.slice(h, 1, T - 1, 1), (R, H))
        else:
            h = b.reshape(h, (R * T, H))
        x = O.rmsnorm(b, h, W("final_norm"), c.norm_eps)
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
