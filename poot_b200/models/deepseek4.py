"""DeepSeek-V4 text stack (crates/poot-models/src/architectures/deepseek4.rs and deepseek4/{stack,sliding,hca,csa,moe}.rs).

The residual stream is ``hc_mult`` parallel streams per token inside manifold-constrained hyper-connection sites
(``components.mhc_pre`` / ``mhc_post``), collapsed by a closing site (``mhc_head``) before the final norm.  Three kinds
of attention layer, chosen per layer by the checkpoint's ``compress_ratios``:

* ``sliding``: the local window over the layer's key-value cache;
* ``hca`` (heavily compressed attention): the window plus every COMPLETE window of a non-overlapping compression of the
  layer's positions;
* ``csa`` (compressed sparse attention): the window plus the best ``index_topk`` entries of an overlapping compression,
  chosen per query token by an indexer with a compressor of its own.

The attention core is not latent attention: a low-rank query with a weightless per-head RMSNorm, ONE key-value head read
as key and as value, interleaved rotary on the trailing ``qk_rope_head_dim`` channels (undone on the output, which
picked up the rotation of the values it read), per-head sink logits and a grouped low-rank output projection.

A compressor turns every ``rate`` consecutive positions into one entry.  The raw key and gate projections of every
position are cached like keys (``cmp_kv_pool`` / ``cmp_gate_pool``) and the entries are recomputed from them each
step - gate plus a learned bias by place in the window, softmax over the window per channel, weighted sum of the keys,
RMSNorm, rotation at the window's first position - so chunks, decode steps and continuations read the same function of
what has been written.  A window is readable once its last position is at or before the query.

Every layer routes through experts scored by ``sqrt(softplus(logit))``; the first ``num_hash_layers`` layers read
their experts from a token-id table instead of ranking them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from ..ir import oplib as O
from ..ir.builder import Builder, Traced
from ..ir.graph import Graph
from ..tensor import DType
from . import components as C
from .config import DecoderConfig, RopeScaling
from .model import Model, StepSpec

F32, I32 = DType.F32, DType.I32


@dataclass
class DeepseekV4Config(DecoderConfig):
    hc_mult: int = 2
    hc_eps: float = 1e-6
    hc_iters: int = 3
    attn_kinds: Optional[List[str]] = None     # "sliding" | "csa" | "hca" per layer
    csa_rate: int = 4
    hca_rate: int = 128
    o_groups: int = 1                           # independent blocks of the first output projection
    o_lora_rank: int = 0
    compress_rope_theta: float = 160000.0       # rotary base of the compressed layers (queries, keys and entries)
    hash_layers: int = 0                        # leading layers whose experts come from the token-id table

    def kind_of(self, l: int) -> str:
        return (self.attn_kinds or ["sliding"] * self.n_layers)[l]

    def rate_of(self, l: int) -> int:
        return {"sliding": 0, "csa": self.csa_rate, "hca": self.hca_rate}[self.kind_of(l)]

    @property
    def in_per_group(self) -> int:
        return self.n_heads * self.head_dim // self.o_groups

    @property
    def prefill_granule(self) -> int:
        """The least common multiple of the compression rates in use: chunks of this many tokens end on window ends."""
        import math
        g = 1
        for k, r in (("csa", self.csa_rate), ("hca", self.hca_rate)):
            if k in (self.attn_kinds or []):
                g = g * r // math.gcd(g, r)
        return g

    def moe_layer(self, l: int) -> bool:
        return True

    def device_gaps(self) -> list:
        return ["hyper-connection residual streams", "compressed attention (window compressors, indexer over compressed entries)",
                "shared key-value head with output de-rotation", "hash-routed experts"]


class DeepseekV4Model(Model):
    """Tracer of the DeepSeek-V4 stack over the standard step contract: one paged pool per layer for the shared
    key-value head, and for a compressed layer the raw key / gate histories of its compressors."""

    def weight_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        H, S, D, nh = c.hidden, c.hc_mult, c.head_dim, c.n_heads
        mix = (2 + S) * S
        s = {"embed": (c.vocab, H), "final_norm": (H,), "lm_head": (c.vocab, H), "hc_head_fn": (S, S * H), "hc_head_base": (S,),
             "hc_head_scale": (1,)}
        for l in range(c.n_layers):
            p = f"layers.{l}."
            s.update({p + "attn_norm": (H,), p + "ffn_norm": (H,)})
            for site in ("attn", "ffn"):
                s.update({p + f"hc_{site}_fn": (mix, S * H), p + f"hc_{site}_base": (mix,), p + f"hc_{site}_scale": (3,)})
            s.update({p + "attn_q_a": (c.q_lora_rank, H), p + "attn_q_a_norm": (c.q_lora_rank,), p + "attn_q_b": (nh * D, c.q_lora_rank),
                      p + "attn_kv": (D, H), p + "attn_kv_norm": (D,), p + "attn_sinks": (nh,),
                      p + "attn_o_a": (c.o_groups * c.o_lora_rank, c.in_per_group), p + "attn_o": (H, c.o_groups * c.o_lora_rank)})
            kind, rate = c.kind_of(l), c.rate_of(l)
            if kind != "sliding":
                raw = D * (2 if kind == "csa" else 1)
                s.update({p + "cmp_kv": (raw, H), p + "cmp_gate": (raw, H), p + "cmp_bias": (rate, raw), p + "cmp_norm": (D,)})
            if kind == "csa":
                ni, di = c.index_n_heads, c.index_head_dim
                s.update({p + "idx_q": (ni * di, c.q_lora_rank), p + "idx_weights": (ni, H), p + "idx_cmp_kv": (2 * di, H),
                          p + "idx_cmp_gate": (2 * di, H), p + "idx_cmp_bias": (rate, 2 * di), p + "idx_cmp_norm": (di,)})
            s.update({p + "ffn_router": (c.n_experts, H), p + "experts_in": (c.n_experts, 2 * c.moe_ffn, H),
                      p + "experts_out": (c.n_experts, H, c.moe_ffn)})
            if l < c.hash_layers:
                s[p + "ffn_hash_table"] = (c.vocab, c.top_k)
            else:
                s[p + "ffn_router_select_bias"] = (c.n_experts,)
            if c.shared_width:
                Fs = c.shared_width
                s.update({p + "shared_gate": (Fs, H), p + "shared_up": (Fs, H), p + "shared_down": (H, Fs)})
        return s

    def trace(self, spec: StepSpec) -> Graph:
        c = self.cfg
        if spec.world != 1:
            raise ValueError(f"{c.family}: no sharding rule for hyper-connection streams")
        if not spec.paged:
            raise ValueError(f"{c.family} is traced over paged pools")
        b = Builder()
        R, T, cap, H, S, D, nh, rot = spec.rows, spec.tokens, spec.capacity, c.hidden, c.hc_mult, c.head_dim, c.n_heads, c.qk_rope_dim
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
        flat_tok, flat_pos = b.reshape(tokens, (L,)), b.reshape(positions, (L,))
        cache = lambda name, rows_: C.paged_cache(b, name, rows_, spec.slots, spec.kv_dtype, write_map, read_map)
        n_pos = max(c.max_position, cap)
        tables: Dict[float, tuple] = {}

        def rope_tables(theta: float):
            if theta not in tables:
                tag = f"rope.{len(tables)}"
                args = (rot, theta, n_pos, RopeScaling())
                tables[theta] = (b.computed(tag + ".cos", (n_pos, rot), F32, "rope_cos", args),
                                 b.computed(tag + ".sin", (n_pos, rot), F32, "rope_sin", args))
            return tables[theta]

        def token_rows(theta: float):
            ct, st = rope_tables(theta)
            return b.reshape(b.gather(ct, flat_pos, 0), (R, T, rot)), b.reshape(b.gather(st, flat_pos, 0), (R, T, rot))

        def window_rows(theta: float, rate: int, n: int):
            """Table rows at positions 0, rate, 2 * rate, ..: where each compressed window starts (known at trace time)."""
            pick = lambda t: b.broadcast(b.reshape(b.slice(b.reshape(b.slice(t, 0, 0, n * rate), (n, rate, rot)), 1, 0, 1), (1, n, rot)), (R, n, rot))
            ct, st = rope_tables(theta)
            return pick(ct), pick(st)

        def complete_windows(rate: int, n: int) -> Traced:
            """I32 ``[R, T, n]``: window ``j`` is readable once its last position ``(j + 1) * rate - 1`` is at or before the query."""
            last = b.iota((R, T, n), 2) * rate + (rate - 1)
            return b.binary("ge", b.broadcast(b.reshape(positions, (R, T, 1)), (R, T, n)), last)

        def overlap_pool(kv: Traced, gate: Traced, entry: int) -> Traced:
            """Entry ``w`` pools the previous window's first-half channels and window ``w``'s second-half channels
            (``2 * rate`` positions); window 0 has no predecessor: zero keys behind a dropped gate (deepseek4/csa.rs)."""
            n = kv.shape[1]
            half = lambda x, i: b.slice(x, 3, i * entry, entry)
            zero = b.slice(half(kv, 0), 1, 0, 1) * 0.0
            dropped = zero + O.MASK_HIDDEN
            prev = lambda x, pad: b.concat([pad, b.slice(half(x, 0), 1, 0, n - 1)], 1) if n > 1 else pad
            return C.softmax_pool(b, b.concat([prev(kv, zero), half(kv, 1)], 2), b.concat([prev(gate, dropped), half(gate, 1)], 2))

        def entries(p: str, tag: str, x: Traced, rate: int, entry: int, overlapping: bool, theta: float) -> Optional[Traced]:
            """A compressor's pooled, normalised and rotated entries ``[R, 1, windows, entry]`` (deepseek4/hca.rs
            ``entries``); this step's raw projections go into the compressor's histories first, at every capacity."""
            raw = entry * (2 if overlapping else 1)
            kv_hist = cache(p + tag + "_kv_pool", O.linear(b, x, W(p + tag + "_kv")))
            gate_hist = cache(p + tag + "_gate_pool", O.linear(b, x, W(p + tag + "_gate")))
            n = cap // rate
            if n == 0:
                return None
            windowed = lambda t: b.reshape(b.slice(t, 2, 0, n * rate), (R, n, rate, raw))
            gate = windowed(gate_hist) + b.broadcast(b.reshape(W(p + tag + "_bias"), (1, 1, rate, raw)), (R, n, rate, raw))
            pooled = overlap_pool(windowed(kv_hist), gate, entry) if overlapping else C.softmax_pool(b, windowed(kv_hist), gate)
            pooled = O.rmsnorm(b, pooled, W(p + tag + "_norm"), c.norm_eps)
            cs, sn = window_rows(theta, rate, n)
            return C.rotate_tail(b, b.reshape(pooled, (R, 1, n, entry)), cs, sn, rot)

        hidden_of = lambda keep: b.select(keep, b.broadcast(b.scalar(0.0, F32), keep.shape), b.broadcast(b.scalar(O.MASK_HIDDEN, F32), keep.shape))

        def attention(l: int, x: Traced) -> Traced:
            p, kind, rate = f"layers.{l}.", c.kind_of(l), c.rate_of(l)
            theta = c.rope_theta if kind == "sliding" else c.compress_rope_theta
            cs, sn = token_rows(theta)
            q_res = norm(O.linear(b, x, W(p + "attn_q_a")), p + "attn_q_a_norm")
            q = b.transpose(b.reshape(O.linear(b, q_res, W(p + "attn_q_b")), (R, T, nh, D)), (0, 2, 1, 3))
            q = q / b.broadcast(b.unary("sqrt", (q * q).sum(-1, keepdim=True) * (1.0 / D) + c.norm_eps), q.shape)
            q = C.rotate_tail(b, q, cs, sn, rot)
            kv = C.rotate_tail(b, b.reshape(norm(O.linear(b, x, W(p + "attn_kv")), p + "attn_kv_norm"), (R, 1, T, D)), cs, sn, rot)
            keys = cache(p + "kv_pool", b.reshape(kv, (L, D)))                                       # [R, 1, cap, D]
            mask = O.causal_mask_from_pos(b, positions, cap, c.sliding_window)                       # [R, T, cap]
            extra = None
            if kind == "hca":
                ent = entries(p, "cmp", x, rate, D, False, theta)
                if ent is not None:
                    extra = (ent, hidden_of(complete_windows(rate, cap // rate)))
            elif kind == "csa":
                ent = entries(p, "cmp", x, rate, D, True, theta)
                index_keys = entries(p, "idx_cmp", x, rate, c.index_head_dim, True, theta)
                if ent is not None:
                    n, ni, di = cap // rate, c.index_n_heads, c.index_head_dim
                    iq = b.transpose(b.reshape(O.linear(b, q_res, W(p + "idx_q")), (R, T, ni, di)), (0, 2, 1, 3))
                    iq = C.rotate_tail(b, iq, cs, sn, rot)
                    kt = b.broadcast(b.transpose(index_keys, (0, 1, 3, 2)), (R, ni, di, n))
                    dots = O.relu(b, b.matmul(iq, kt, "exact")) * (di ** -0.5)                    # [R, ni, T, n]
                    hw = O.linear(b, x, W(p + "idx_weights"), precision="exact") * (ni ** -0.5)
                    hw = b.reshape(b.transpose(b.reshape(hw, (R, T, ni)), (0, 2, 1)), (R, ni, T, 1))
                    readable = complete_windows(rate, n)
                    ranked = (dots * b.broadcast(hw, dots.shape)).sum(1) + hidden_of(readable)
                    # windows tied at the cut are all kept: the rank counts strictly greater scores only
                    best = O.lnot(b, b.binary("ge", C.pairwise_rank(b, ranked), b.broadcast(b.scalar(min(c.index_topk, n), I32), (R, T, n))))
                    extra = (ent, hidden_of(b.binary("and", best, readable)))
            if extra is not None:
                keys, mask = b.concat([keys, extra[0]], 2), b.concat([mask, extra[1]], 2)
            out = O.attention_biased(b, q, keys, keys, mask, D ** -0.5, nh, 0.0, None, W(p + "attn_sinks"))
            out = C.rotate_tail(b, out, cs, sn, rot, inverse=True)        # the values carried their positions' rotation
            G, ipg, r_o = c.o_groups, c.in_per_group, c.o_lora_rank
            groups = b.transpose(b.reshape(b.transpose(out, (0, 2, 1, 3)), (L, G, ipg)), (1, 0, 2))
            blocks = b.transpose(b.reshape(W(p + "attn_o_a"), (G, r_o, ipg)), (0, 2, 1))
            mixed = b.reshape(b.transpose(b.matmul(groups, blocks), (1, 0, 2)), (L, G * r_o))
            return O.linear(b, mixed, W(p + "attn_o"))

        def ffn(l: int, x: Traced) -> Traced:
            p = f"layers.{l}."
            hashed = l < c.hash_layers
            ids = None
            if hashed:
                table = b.input(p + "ffn_hash_table", shapes[p + "ffn_hash_table"], I32, storage="const", range=(0, c.n_experts - 1))
                ids = b.gather(table, flat_tok, 0)                                                  # [L, top_k]
            f = O.moe_routed(b, x, W(p + "ffn_router"), W(p + "experts_in"), W(p + "experts_out"), c.top_k, score="sqrtsoftplus",
                             renorm=True, select_bias=None if hashed else W(p + "ffn_router_select_bias"),
                             routed_scale=c.routed_scale, act="silu_clamped", limit=c.swiglu_limit, route_ids=ids)
            if c.shared_width:
                a = O.ffn_activation(b, O.linear(b, x, W(p + "shared_gate")), O.linear(b, x, W(p + "shared_up")), "silu_clamped",
                                     c.swiglu_limit)
                f = f + O.linear(b, a, W(p + "shared_down"))
            return f

        xs = C.mhc_widen(b, b.gather(W("embed"), flat_tok, 0), S)
        for l in range(c.n_layers):
            p = f"layers.{l}."
            for site, block, nrm in (("attn", attention, "attn_norm"), ("ffn", ffn, "ffn_norm")):
                x, post, comb = C.mhc_pre(b, xs, W(p + f"hc_{site}_fn"), W(p + f"hc_{site}_base"), W(p + f"hc_{site}_scale"),
                                          c.norm_eps, c.hc_eps, c.hc_iters)
                xs = C.mhc_post(b, post, comb, block(l, norm(x, p + nrm)), xs)
        if spec.logit_rows == "last":
            xs = b.reshape(b.slice(b.reshape(xs, (R, T, S, H)), 1, T - 1, 1), (R, S, H))
        h = C.mhc_head(b, xs, W("hc_head_fn"), W("hc_head_base"), W("hc_head_scale"), c.norm_eps, c.hc_eps)
        x = norm(h, "final_norm")
        if spec.carry:
            b.output(x, "hidden", "export")
        logits = O.linear(b, x, W("lm_head"))
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
