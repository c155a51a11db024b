"""Gemma 4 text stack (crates/poot-models/src/architectures: the gemma4 entry with ``ple.rs`` per-layer embeddings and
the proportional rotary table).

What sets the layer apart from the standard stack, and why it has a tracer of its own:

* head width and K/V head count differ by layer type: full-attention layers use ``global_head_dim`` (and, with
  ``k_eq_v``, ``n_global_kv_heads`` heads whose value is the key projection itself); scores are not scaled; q and k get a
  per-head RMSNorm with a weight, v one without;
* full-attention layers rotate only the first share of the head's ``(i, i + D/2)`` channel pairs (proportional rope:
  the table spans the whole head, the other pairs have frequency 0); windowed layers use the default table;
* the last ``kv_shared_layers`` layers compute no keys or values: each attends over the K/V of the last earlier layer of
  its own type (and may have a double-width FFN);
* every projection's output passes an RMSNorm before its residual add (sandwich block); with ``moe_block`` the FFN is
  a dense FFN plus routed experts, each behind its own norms, the router reading the un-normed residual through a
  weightless RMSNorm, a learned scale and ``hidden ** -0.5``, and scaling each expert's gate by a learned factor;
* per-layer embeddings: a second table gives every token ``n_layers * ple_dim`` values, averaged with a projection of
  the token's embedding; layer ``l`` gates its slice into the residual stream after the FFN;
* each layer ends by scaling the residual stream with a stored scalar.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

from ..ir import oplib as O
from ..ir.builder import Builder, Traced
from ..ir.graph import Graph
from ..tensor import DType
from .config import DecoderConfig, RopeScaling
from .model import Model, StepSpec

F32, I32 = DType.F32, DType.I32


@dataclass
class Gemma4Config(DecoderConfig):
    global_head_dim: int = 0           # head width of full-attention layers (0: head_dim)
    n_global_kv_heads: int = 0         # K/V heads of full-attention layers under k_eq_v (0: n_kv_heads)
    k_eq_v: bool = False               # full-attention layers have no value projection: v is the key projection
    kv_shared_layers: int = 0          # trailing layers that reuse an earlier layer's K/V
    double_wide_mlp: bool = False      # K/V-sharing layers have a dense FFN of twice the width
    ple_dim: int = 0                   # per-layer embedding width (0: none)
    ple_vocab: int = 0
    moe_block: bool = False            # dense FFN + routed experts in every layer
    rope_proportion: float = 1.0       # share of a full-attention head's channel pairs that rotate

    def is_full(self, l: int) -> bool:
        return self.window_of(l) == 0

    def head_dim_of(self, l: int) -> int:
        return self.global_head_dim if (self.is_full(l) and self.global_head_dim) else self.head_dim

    def kv_heads_of(self, l: int) -> int:
        return self.n_global_kv_heads if (self.k_eq_v and self.is_full(l) and self.n_global_kv_heads) else self.n_kv_heads

    def value_is_key(self, l: int) -> bool:
        return self.k_eq_v and self.is_full(l)

    @property
    def first_shared(self) -> int:
        return self.n_layers - self.kv_shared_layers

    def kv_source(self, l: int) -> Optional[int]:
        """Layer whose K/V layer ``l`` attends over (``None``: its own)."""
        fs = self.first_shared
        if not (l >= fs > 0):
            return None
        for j in range(fs - 1, -1, -1):
            if self.is_full(j) == self.is_full(l):
                return j
        raise ValueError(f"layer {l} shares K/V but no earlier layer has its attention type")

    def ffn_of(self, l: int) -> int:
        return self.ffn * (2 if (self.double_wide_mlp and l >= self.first_shared > 0) else 1)

    def device_gaps(self) -> list:
        return ["gemma4 layer (head widths by layer type, K/V shared between layers, per-layer embeddings, proportional rope)"]


class Gemma4Model(Model):
    """Tracer of the Gemma 4 text stack over the same step contract as ``Model`` (tokens, positions, read / write maps,
    paged K/V pools per K/V-owning layer, logits)."""

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H = c.hidden
        s = {"embed": (c.vocab, H), "final_norm": (H,)}
        if c.ple_dim:
            s.update({"ple_embed": (c.ple_vocab, c.n_layers * c.ple_dim), "ple_model_proj": (c.n_layers * c.ple_dim, H),
                      "ple_proj_norm": (c.ple_dim,)})
        for l in range(c.n_layers):
            p = f"layers.{l}."
            D, nkv = c.head_dim_of(l), c.kv_heads_of(l)
            s.update({p + "attn_norm": (H,), p + "attn_post_norm": (H,), p + "ffn_norm": (H,), p + "ffn_post_norm": (H,),
                      p + "attn_q": (c.n_heads * D, H), p + "attn_q_norm": (D,), p + "attn_o": (H, c.n_heads * D),
                      p + "layer_scalar": (1,)})
            if c.kv_source(l) is None:
                s.update({p + "attn_k": (nkv * D, H), p + "attn_k_norm": (D,)})
                if not c.value_is_key(l):
                    s[p + "attn_v"] = (nkv * D, H)
            F = c.ffn_of(l)
            s.update({p + "ffn_gate": (F, H), p + "ffn_up": (F, H), p + "ffn_down": (H, F)})
            if c.moe_block:
                s.update({p + "ffn_post_norm_1": (H,), p + "ffn_norm_2": (H,), p + "ffn_post_norm_2": (H,),
                          p + "ffn_router": (c.n_experts, H), p + "ffn_router_scale": (H,),
                          p + "ffn_expert_scale": (c.n_experts,), p + "experts_in": (c.n_experts, 2 * c.moe_ffn, H),
                          p + "experts_out": (c.n_experts, H, c.moe_ffn)})
            if c.ple_dim:
                s.update({p + "ple_gate": (c.ple_dim, H), p + "ple_proj": (H, c.ple_dim), p + "ple_post_norm": (H,)})
        return s

    def trace(self, spec: StepSpec) -> Graph:
        c = self.cfg
        if spec.world != 1:
            raise ValueError("gemma4: no sharding rule for layers that share K/V")
        if not spec.paged:
            raise ValueError("gemma4 is traced over paged K/V pools")
        b = Builder()
        R, T, cap, H, Hq = spec.rows, spec.tokens, spec.capacity, c.hidden, c.n_heads
        L = R * T
        shapes = self.weight_shapes()
        consts: Dict[str, Traced] = {}

        def W(name: str) -> Traced:
            if name not in consts:
                consts[name] = b.const(name, shapes[name], spec.weight_dtype).cast(F32)
            return consts[name]

        def norm(x: Traced, name: Optional[str]) -> Traced:
            """RMSNorm over the last axis; ``None``: without a weight."""
            D = x.shape[-1]
            den = b.unary("sqrt", (x * x).sum(-1, keepdim=True) * (1.0 / D) + c.norm_eps)
            y = x / b.broadcast(den, x.shape)
            return y * b.broadcast(W(name), x.shape) if name is not None else y

        tokens = b.slot("tokens", (R, T), I32, "token", range=(0, c.vocab - 1))
        positions = b.slot("positions", (R, T), I32, "pos", range=(0, c.max_position - 1))
        read_map = b.slot("read_map", (R, cap), I32, "slot_map", range=(0, spec.slots - 1))
        write_map = b.slot("write_map", (L,), I32, "write_map", range=(-1, spec.slots - 1))
        flat_pos = b.reshape(positions, (L,))
        flat_tok = b.reshape(tokens, (L,))

        ropes: Dict[bool, tuple] = {}

        def rope_of(l: int):
            full = c.is_full(l)
            if full not in ropes:
                D = c.head_dim_of(l)
                theta = c.rope_theta if full else (c.rope_theta_local or c.rope_theta)
                scaling = RopeScaling(kind="proportional", proportion=c.rope_proportion) if full else RopeScaling()
                tag = "rope" if full else "rope.local"
                ct = b.computed(tag + ".cos", (c.max_position, D), F32, "rope_cos", (D, theta, c.max_position, scaling))
                st = b.computed(tag + ".sin", (c.max_position, D), F32, "rope_sin", (D, theta, c.max_position, scaling))
                ropes[full] = (b.gather(ct, flat_pos, 0), b.gather(st, flat_pos, 0))
            return ropes[full]

        masks: Dict[int, Traced] = {}

        def mask_of(l: int) -> Traced:
            win = c.window_of(l)
            if win not in masks:
                masks[win] = O.causal_mask_from_pos(b, positions, cap, win)
            return masks[win]

        h = b.gather(W("embed"), flat_tok, 0) * math.sqrt(H)
        if spec.embeds:
            rows_in = b.slot("embed_rows", (L, H), F32, "activation")
            flagged = b.slot("embed_flags", (L,), I32, "activation", range=(0, 1))
            h = b.select(b.broadcast(b.reshape(flagged, (L, 1)), (L, H)), rows_in, h)
        per_layer = None
        if c.ple_dim:
            P, NL = c.ple_dim, c.n_layers
            from_table = b.reshape(b.gather(W("ple_embed"), flat_tok, 0) * math.sqrt(P), (L, NL, P))
            from_model = b.reshape(O.linear(b, h, W("ple_model_proj")) * (H ** -0.5), (L, NL, P))
            per_layer = (norm(from_model, "ple_proj_norm") + from_table) * (2.0 ** -0.5)

        kv_views: Dict[int, tuple] = {}
        for l in range(c.n_layers):
            p = f"layers.{l}."
            D, nkv = c.head_dim_of(l), c.kv_heads_of(l)
            cos, sin = rope_of(l)
            x = norm(h, p + "attn_norm")
            q = b.reshape(O.linear(b, x, W(p + "attn_q")), (L, Hq, D))
            q = O.rope(b, norm(q, p + "attn_q_norm"), cos, sin, D)
            src = c.kv_source(l)
            if src is None:
                k = b.reshape(O.linear(b, x, W(p + "attn_k")), (L, nkv, D))
                v = k if c.value_is_key(l) else b.reshape(O.linear(b, x, W(p + "attn_v")), (L, nkv, D))
                k = O.rope(b, norm(k, p + "attn_k_norm"), cos, sin, D)
                v = norm(v, None)
                kp = b.state(p + "k_pool", (spec.slots, nkv, D), spec.kv_dtype, "blocked").cast(F32)
                vp = b.state(p + "v_pool", (spec.slots, nkv, D), spec.kv_dtype, "blocked").cast(F32)
                kp2, vp2 = b.scatter_update(kp, write_map, k), b.scatter_update(vp, write_map, v)
                b.output(kp2.cast(spec.kv_dtype), p + "k_pool.next", "state_next", p + "k_pool")
                b.output(vp2.cast(spec.kv_dtype), p + "v_pool.next", "state_next", p + "v_pool")
                kv_views[l] = (O.paged_view(b, kp2.cast(spec.kv_dtype).cast(F32), read_map),
                               O.paged_view(b, vp2.cast(spec.kv_dtype).cast(F32), read_map))
                src = l
            Kv, Vv = kv_views[src]
            qh = b.transpose(b.reshape(q, (R, T, Hq, D)), (0, 2, 1, 3))
            a = O.attention_masked(b, qh, Kv, Vv, mask_of(l), 1.0, Hq // nkv, 0.0)
            a = b.reshape(b.transpose(a, (0, 2, 1, 3)), (L, Hq * D))
            h = h + norm(O.linear(b, a, W(p + "attn_o")), p + "attn_post_norm")

            x = norm(h, p + "ffn_norm")
            f = O.linear(b, O.ffn_activation(b, O.linear(b, x, W(p + "ffn_gate")), O.linear(b, x, W(p + "ffn_up")), c.act),
                         W(p + "ffn_down"))
            if c.moe_block:
                routed_in = norm(h, None) * b.broadcast(W(p + "ffn_router_scale"), (L, H)) * (H ** -0.5)
                routed = O.moe_routed(b, norm(h, p + "ffn_norm_2"), W(p + "ffn_router"), W(p + "experts_in"),
                                      W(p + "experts_out"), c.top_k, score="softmax", renorm=True, act=c.act,
                                      router_x=routed_in, expert_scale=W(p + "ffn_expert_scale"))
                f = norm(f, p + "ffn_post_norm_1") + norm(routed, p + "ffn_post_norm_2")
            h = h + norm(f, p + "ffn_post_norm")
            if c.ple_dim:
                mine = b.reshape(b.slice(per_layer, 1, l, 1), (L, c.ple_dim))
                g = O.ffn_activation(b, O.linear(b, h, W(p + "ple_gate")), mine, c.act)
                h = h + norm(O.linear(b, g, W(p + "ple_proj")), p + "ple_post_norm")
            h = h * b.broadcast(b.reshape(W(p + "layer_scalar"), (1, 1)), (L, H))

        h = b.reshape(h, (R, T, H))
        h = b.reshape(b.slice(h, 1, T - 1, 1), (R, H)) if spec.logit_rows == "last" else b.reshape(h, (L, H))
        logits = O.linear(b, norm(h, "final_norm"), W("embed") if c.tie_embeddings else W("lm_head"))
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
