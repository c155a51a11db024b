"""GLM-5.3-Flash text stack (crates/poot-models/src/architectures/glm53_flash.rs, glm53_flash/stack.rs, mtp.rs).

The residual stream of a token is ``hc_mult`` parallel streams.  Every block - the token mixer and the feed-forward of
each layer - sits inside a manifold-constrained hyper-connection site (``components.mhc_pre`` / ``mhc_post``): the site
collapses the streams into the block's input, places the block's output back on each stream and mixes the old streams
with a near doubly-stochastic matrix.  The stack ends with the MEAN of the streams under the closing norm.

Two token mixers, chosen per layer by the checkpoint's ``layer_types``:

* ``kda``: Kimi delta attention, a gated delta rule over a carried matrix state with a decay per key channel;
* ``dsa``: latent attention without a rotary part under a pooled indexer's keep mask.

The feed-forward is a dense gated block or a shared expert plus routed experts behind the sigmoid router with a
selection-only bias; both gate with the clamped SwiGLU ``silu(min(g, limit)) * clamp(u, -limit, limit)``.

The checkpoint's multi-token-prediction layer is a one-block model of its own (``Glm53Model.mtp_model``): a ``dsa``
block with plain pre-norm residuals (no hyper-connection sites) behind ``eh_proj [enorm(embed) ; hnorm(carry)]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional

from ..ir import oplib as O
from ..ir.builder import Builder, Traced
from ..ir.graph import Graph
from ..tensor import DType
from . import components as C
from .config import DecoderConfig
from .model import Model, StepSpec

F32, I32 = DType.F32, DType.I32


@dataclass
class Glm53Config(DecoderConfig):
    hc_mult: int = 2                    # residual streams per token
    hc_eps: float = 1e-6                # floor after every sigmoid / softmax / Sinkhorn division of a site
    hc_iters: int = 3                   # Sinkhorn rounds
    ffn_kinds: Optional[List[str]] = None   # "dense" | "sparse" per layer
    kda_heads: int = 0
    kda_head_dim: int = 0
    kda_conv: int = 4
    kda_lower_bound: float = -5.0       # the log forget gate lies in (lower_bound, 0)
    index_kpool: int = 1                # positions pooled into one indexer key
    hyper: bool = True                  # False: plain residuals (the multi-token-prediction layer)

    @property
    def is_recurrent(self) -> bool:
        return any(k == "kda" for k in (self.layer_kinds or []))

    def ffn_kind(self, l: int) -> str:
        return (self.ffn_kinds or ["sparse"] * self.n_layers)[l]

    def moe_layer(self, l: int) -> bool:
        return self.ffn_kind(l) == "sparse"

    @property
    def mix(self) -> int:
        return (2 + self.hc_mult) * self.hc_mult

    def device_gaps(self) -> list:
        return ["hyper-connection residual streams", "kimi delta attention", "latent attention under a pooled indexer"]


class Glm53Model(Model):
    """Tracer of the GLM-5.3-Flash text stack over the standard step contract (tokens, positions, read / write maps,
    paged pools for the latent and indexer caches, recurrent state rows for the delta-rule layers, logits)."""

    def mtp_model(self) -> "Glm53Model":
        c = self.cfg
        if c.mtp_layers != 1:
            # the reference cycles several layers by draft step, which a step shape does not name
            raise ValueError(f"{c.family} stores {c.mtp_layers} multi-token-prediction layers; the draft program traces exactly one")
        return Glm53Model(replace(c, name=c.name + "-mtp", n_layers=1, layer_kinds=["dsa"], ffn_kinds=[c.ffn_kind(c.n_layers - 1)],
                                  mtp_layers=0, mtp_head=True, hyper=False))

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H, S = c.hidden, c.hc_mult
        s = {"embed": (c.vocab, H), "final_norm": (H,)}
        if not c.tie_embeddings:
            s["lm_head"] = (c.vocab, H)
        if c.mtp_head:
            s.update({"mtp.enorm": (H,), "mtp.hnorm": (H,), "mtp.eh_proj": (H, 2 * H)})
        for l in range(c.n_layers):
            p = f"layers.{l}."
            s.update({p + "attn_norm": (H,), p + "ffn_norm": (H,)})
            if c.hyper:
                for site in ("attn", "ffn"):
                    s.update({p + f"hc_{site}_fn": (c.mix, S * H), p + f"hc_{site}_base": (c.mix,), p + f"hc_{site}_scale": (3,)})
            if c.mixer_of(l) == "kda":
                h, d, K = c.kda_heads, c.kda_head_dim, c.kda_conv
                Cw = h * d
                s.update({p + "kda_q": (Cw, H), p + "kda_k": (Cw, H), p + "kda_v": (Cw, H), p + "kda_conv_q": (Cw, K),
                          p + "kda_conv_k": (Cw, K), p + "kda_conv_v": (Cw, K), p + "kda_f_a": (d, H), p + "kda_f_b": (Cw, d),
                          p + "kda_b": (h, H), p + "kda_g_a": (d, H), p + "kda_g_b": (Cw, d), p + "kda_a_log": (h,),
                          p + "kda_dt_bias": (Cw,), p + "kda_o_norm": (d,), p + "kda_o": (H, Cw)})
            else:
                nh, qk, vd, ni, di = c.n_heads, c.qk_nope_dim, c.v_head_dim, c.index_n_heads, c.index_head_dim
                s.update({p + "attn_q_a": (c.q_lora_rank, H), p + "attn_q_a_norm": (c.q_lora_rank,),
                          p + "attn_q_b": (nh * qk, c.q_lora_rank), p + "attn_kv_a": (c.kv_lora_rank, H),
                          p + "attn_kv_a_norm": (c.kv_lora_rank,), p + "attn_kv_b": (nh * (qk + vd), c.kv_lora_rank),
                          p + "attn_o": (H, nh * vd), p + "idx_q": (ni * di, c.q_lora_rank), p + "idx_k": (di, H),
                          p + "idx_k_norm": (di,), p + "idx_k_norm_bias": (di,), p + "idx_weights": (ni, H),
                          p + "idx_pool_gate": (di, H), p + "idx_pool_bias": (c.index_kpool, di)})
            if c.ffn_kind(l) == "dense":
                s.update({p + "ffn_gate": (c.ffn, H), p + "ffn_up": (c.ffn, H), p + "ffn_down": (H, c.ffn)})
            else:
                Fs = c.shared_width
                s.update({p + "ffn_router": (c.n_experts, H), p + "ffn_router_select_bias": (c.n_experts,),
                          p + "experts_in": (c.n_experts, 2 * c.moe_ffn, H), p + "experts_out": (c.n_experts, H, c.moe_ffn)})
                if Fs:
                    s.update({p + "shared_gate": (Fs, H), p + "shared_up": (Fs, H), p + "shared_down": (H, Fs)})
        return s

    def trace(self, spec: StepSpec) -> Graph:
        c = self.cfg
        if spec.world != 1:
            raise ValueError(f"{c.family}: no sharding rule for hyper-connection streams")
        if not spec.paged:
            raise ValueError(f"{c.family} is traced over paged pools")
        b = Builder()
        R, T, cap, H, S = spec.rows, spec.tokens, spec.capacity, c.hidden, c.hc_mult
        L = R * T
        shapes = self.weight_shapes()
        consts: Dict[str, Traced] = {}

        def W(name: str) -> Traced:
            if name not in consts:
                consts[name] = b.const(name, shapes[name], spec.weight_dtype).cast(F32)
            return consts[name]

        norm = lambda x, name: O.rmsnorm(b, x, W(name), c.norm_eps)
        tokens = b.slot("tokens", (R, T), I32, "token", range=(0, c.vocab - 1))
        positions = b.slot("positions", (R, T), I32, "pos", range=(0, c.max_position - 1))
        read_map = b.slot("read_map", (R, cap), I32, "slot_map", range=(0, spec.slots - 1))
        write_map = b.slot("write_map", (L,), I32, "write_map", range=(-1, spec.slots - 1))

        def mixer(l: int, x: Traced) -> Traced:
            p = f"layers.{l}."
            if c.mixer_of(l) == "kda":
                return C.kda_mixer(b, x, W, p, R, T, c.kda_heads, c.kda_head_dim, c.kda_conv, c.kda_lower_bound, c.norm_eps)
            return C.pooled_dsa(b, x, W, p, positions, read_map, write_map, spec.slots, spec.kv_dtype, c.n_heads, c.qk_nope_dim,
                                c.v_head_dim, c.kv_lora_rank, c.norm_eps, c.index_n_heads, c.index_head_dim, c.index_kpool,
                                c.index_topk // c.index_kpool)

        def glu_ffn(x: Traced, p: str, gate: str, up: str, down: str) -> Traced:
            a = O.ffn_activation(b, O.linear(b, x, W(p + gate)), O.linear(b, x, W(p + up)), "silu_clamped", c.swiglu_limit)
            return O.linear(b, a, W(p + down))

        def ffn(l: int, x: Traced) -> Traced:
            p = f"layers.{l}."
            if c.ffn_kind(l) == "dense":
                return glu_ffn(x, p, "ffn_gate", "ffn_up", "ffn_down")
            f = O.moe_routed(b, x, W(p + "ffn_router"), W(p + "experts_in"), W(p + "experts_out"), c.top_k, score="sigmoid",
                             renorm=c.norm_topk_prob, select_bias=W(p + "ffn_router_select_bias"), n_group=c.n_group,
                             topk_group=c.topk_group, routed_scale=c.routed_scale, act="silu_clamped", limit=c.swiglu_limit)
            return f + glu_ffn(x, p, "shared_gate", "shared_up", "shared_down") if c.shared_width else f

        h = b.gather(W("embed"), b.reshape(tokens, (L,)), 0)
        if c.mtp_head:
            # the embedding of the token that follows a position (zero at absolute position 0) and the target's closing
            # hidden state of that position, each under its own norm, embedding first (glm53_flash/mtp.rs:9-13)
            carry = b.slot("carry", (L, H), F32, "activation")
            first = b.binary("ge", b.broadcast(b.scalar(0, I32), (L, 1)), b.reshape(positions, (L, 1)))
            h = b.select(b.broadcast(first, (L, H)), b.broadcast(b.scalar(0.0, F32), (L, H)), h)
            h = O.linear(b, b.concat([norm(h, "mtp.enorm"), norm(carry, "mtp.hnorm")], -1), W("mtp.eh_proj"))
        if c.hyper:
            xs = C.mhc_widen(b, h, S)
            for l in range(c.n_layers):
                p = f"layers.{l}."
                for site, block, nrm in (("attn", mixer, "attn_norm"), ("ffn", ffn, "ffn_norm")):
                    x, post, comb = C.mhc_pre(b, xs, W(p + f"hc_{site}_fn"), W(p + f"hc_{site}_base"), W(p + f"hc_{site}_scale"),
                                              c.norm_eps, c.hc_eps, c.hc_iters)
                    xs = C.mhc_post(b, post, comb, block(l, norm(x, p + nrm)), xs)
            h = xs.sum(1) * (1.0 / S)
        else:
            for l in range(c.n_layers):
                p = f"layers.{l}."
                h = h + mixer(l, norm(h, p + "attn_norm"))
                h = h + ffn(l, norm(h, p + "ffn_norm"))
        h = b.reshape(h, (R, T, H))
        h = b.reshape(b.slice(h, 1, T - 1, 1), (R, H)) if spec.logit_rows == "last" else b.reshape(h, (L, H))
        x = norm(h, "final_norm")
        if spec.carry or c.mtp_head:
            b.output(x, "hidden", "export")
        logits = O.linear(b, x, W("embed") if c.tie_embeddings else W("lm_head"))
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
