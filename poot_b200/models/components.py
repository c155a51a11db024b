"""Trace components shared by the families with a tracer of their own: manifold-constrained hyper-connections, the
Kimi delta attention mixer and latent attention under a pooled indexer.

Every function takes the builder and flat token rows (``[L, ...]`` with ``L = rows * tokens``, row-major by sequence
row) and emits primitive equations plus the step's state reads / writes, like the standard tracer's closures.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

from ..ir import oplib as O
from ..ir.builder import Builder, Traced
from ..tensor import DType

F32, I32 = DType.F32, DType.I32


# ---- manifold-constrained hyper-connections ----------------------------------------------------------------------
def mhc_widen(b: Builder, h: Traced, streams: int) -> Traced:
    """``[L, H] -> [L, streams, H]``: every residual stream starts as a copy of the embedding
    (crates/poot-models/src/components/mhc.rs ``widen``)."""
    L, H = h.shape
    return b.broadcast(b.reshape(h, (L, 1, H)), (L, streams, H))


def _mhc_mix(b: Builder, xs: Traced, fn: Traced, eps: float) -> Traced:
    L, S, H = xs.shape
    flat = b.reshape(xs, (L, S * H))
    den = b.unary("sqrt", (flat * flat).sum(-1, keepdim=True) * (1.0 / (S * H)) + eps)
    return O.linear(b, flat / b.broadcast(den, flat.shape), fn, precision="exact")


def _mhc_collapse(b: Builder, xs: Traced, pre: Traced) -> Traced:
    L, S, H = xs.shape
    return (xs * b.broadcast(b.reshape(pre, (L, S, 1)), xs.shape)).sum(1)


def mhc_pre(b: Builder, xs: Traced, fn: Traced, base: Traced, scale: Traced, eps: float, hc_eps: float,
            iters: int) -> Tuple[Traced, Traced, Traced]:
    """One hyper-connection site over the widened streams ``xs[L, S, H]`` (components/mhc.rs ``mhc_pre``): the
    RMS-normalised concatenation of a token's streams is projected by ``fn[(2 + S) * S, S * H]`` into three groups of
    logits, each scaled by its entry of ``scale[3]`` and shifted by ``base``:

    * ``pre[L, S]  = sigmoid(.) + hc_eps``: weights collapsing the streams into the block's input;
    * ``post[L, S] = 2 * sigmoid(.)``: weights placing the block's output back on every stream;
    * ``comb[L, S, S]``: ``softmax(.) + hc_eps`` over the last axis, projected towards the doubly stochastic matrices
      by Sinkhorn-Knopp: one column normalisation, then ``iters - 1`` rounds of rows and columns, every division by
      ``sum + hc_eps``.

    Returns ``(collapsed[L, H], post, comb)``."""
    L, S, H = xs.shape
    mix = _mhc_mix(b, xs, fn, eps)

    def group(lo: int, n: int, which: int, shape) -> Traced:
        w = b.reshape(b.slice(mix, -1, lo, n), (L,) + shape)
        s = b.broadcast(b.reshape(b.slice(scale, 0, which, 1), (1,) * (1 + len(shape))), w.shape)
        return w * s + b.broadcast(b.reshape(b.slice(base, 0, lo, n), (1,) + shape), w.shape)

    pre = O.sigmoid(b, group(0, S, 0, (S,))) + hc_eps
    post = O.sigmoid(b, group(S, S, 1, (S,))) * 2.0
    comb = O.softmax(b, group(2 * S, S * S, 2, (S, S))) + hc_eps
    cols = lambda m: m / b.broadcast(m.sum(1, keepdim=True) + hc_eps, m.shape)
    rows = lambda m: m / b.broadcast(m.sum(-1, keepdim=True) + hc_eps, m.shape)
    comb = cols(comb)
    for _ in range(1, iters):
        comb = cols(rows(comb))
    return _mhc_collapse(b, xs, pre), post, comb


def mhc_post(b: Builder, post: Traced, comb: Traced, out: Traced, xs: Traced) -> Traced:
    """The widened streams after a block: ``post[s] * out`` on stream ``s`` plus the old streams mixed by the transpose
    of ``comb`` (stream ``s`` receives ``sum_j comb[j, s] * xs[j]``; components/mhc.rs ``mhc_post``)."""
    L, S, H = xs.shape
    placed = b.broadcast(b.reshape(post, (L, S, 1)), xs.shape) * b.broadcast(b.reshape(out, (L, 1, H)), xs.shape)
    return placed + b.matmul(b.transpose(comb, (0, 2, 1)), xs, "exact")


def mhc_head(b: Builder, xs: Traced, fn: Traced, base: Traced, scale: Traced, eps: float, hc_eps: float) -> Traced:
    """The closing collapse of a model that ends with a site's ``pre`` alone: ``fn[S, S * H]``, ``base[S]``,
    ``scale[1]`` (components/mhc.rs ``mhc_head``)."""
    L, S, H = xs.shape
    mix = _mhc_mix(b, xs, fn, eps)
    logits = mix * b.broadcast(b.reshape(scale, (1, 1)), mix.shape) + b.broadcast(b.reshape(base, (1, S)), mix.shape)
    return _mhc_collapse(b, xs, O.sigmoid(b, logits) + hc_eps)


# ---- Kimi delta attention ----------------------------------------------------------------------------------------
def kda_mixer(b: Builder, x: Traced, W: Callable[[str], Traced], p: str, R: int, T: int, heads: int, dim: int,
              kernel: int, lower_bound: float, eps: float) -> Traced:
    """The KDA mixer over ``x[L, H]`` (crates/poot-models/src/components/kda.rs): query, key and value projections ->
    causal depthwise conv + SiLU over each -> unit-norm query (scaled by ``dim ** -0.5``) and key per head -> the
    gated delta rule per head with a decay PER KEY CHANNEL,

        ``g = lower_bound * sigmoid(exp(a_log) * (f_b(f_a(x)) + dt_bias))``      (log decay, in ``(lower_bound, 0)``)
        ``S = exp(g)[:, None] * S;  d = beta * (v - S^T k);  S = S + outer(k, d);  o = S^T q``

    -> RMSNorm per head with ``o_norm`` gated by ``sigmoid(g_b(g_a(x)))`` -> out projection.  The three conv windows are
    carried as one ``[K - 1, 3 * heads * dim]`` state per sequence row (query channels, then key, then value) and the
    matrix state as ``[heads, dim, dim]`` (key channel, then value channel)."""
    L = R * T
    C = heads * dim
    mixed = b.concat([O.linear(b, x, W(p + "kda_q")), O.linear(b, x, W(p + "kda_k")), O.linear(b, x, W(p + "kda_v"))], -1)
    taps = b.concat([W(p + "kda_conv_q"), W(p + "kda_conv_k"), W(p + "kda_conv_v")], 0)              # [3C, K]
    f = O.linear(b, O.linear(b, x, W(p + "kda_f_a")), W(p + "kda_f_b")) + b.broadcast(W(p + "kda_dt_bias"), (L, C))
    rate = b.broadcast(b.reshape(b.unary("exp", W(p + "kda_a_log")), (1, heads, 1)), (L, heads, dim))
    g = O.sigmoid(b, rate * b.reshape(f, (L, heads, dim))) * lower_bound                             # [L, heads, dim]
    beta = O.sigmoid(b, O.linear(b, x, W(p + "kda_b")))                                              # [L, heads]
    conv_in = b.state(p + "conv_state", (R, kernel - 1, 3 * C), F32, "recurrent")
    s_in = b.state(p + "kda_state", (R, heads, dim, dim), F32, "recurrent")
    ys, convs, states = [], [], []
    for r in range(R):
        y, cs = O.causal_conv1d(b, b.slice(mixed, 0, r * T, T), b.reshape(b.slice(conv_in, 0, r, 1), (kernel - 1, 3 * C)), taps)
        y = O.silu(b, y)
        by_head = lambda t: b.transpose(b.reshape(t, (1, T, heads, t.shape[-1] // heads)), (0, 2, 1, 3))
        q = O.l2norm(b, by_head(b.slice(y, 1, 0, C))) * (1.0 / math.sqrt(dim))
        k = O.l2norm(b, by_head(b.slice(y, 1, C, C)))
        v = by_head(b.slice(y, 1, 2 * C, C))
        gr = b.transpose(b.reshape(b.slice(g, 0, r * T, T), (1, T, heads, dim)), (0, 2, 1, 3))
        br = b.reshape(b.transpose(b.slice(beta, 0, r * T, T), (1, 0)), (1, heads, T, 1))
        yo, so = b.scan("delta_rule", [q, k, v, gr, br, b.slice(s_in, 0, r, 1)])
        ys.append(b.reshape(b.transpose(yo, (0, 2, 1, 3)), (T, heads, dim)))
        convs.append(b.reshape(cs, (1, kernel - 1, 3 * C)))
        states.append(so)
    b.output(b.concat(convs, 0) if R > 1 else convs[0], p + "conv_state.next", "state_next", p + "conv_state")
    b.output(b.concat(states, 0) if R > 1 else states[0], p + "kda_state.next", "state_next", p + "kda_state")
    y = b.concat(ys, 0) if R > 1 else ys[0]
    gate = O.sigmoid(b, b.reshape(O.linear(b, O.linear(b, x, W(p + "kda_g_a")), W(p + "kda_g_b")), (L, heads, dim)))
    out = O.rmsnorm(b, y, W(p + "kda_o_norm"), eps) * gate
    return O.linear(b, b.reshape(out, (L, C)), W(p + "kda_o"))


# ---- latent attention under a pooled indexer -----------------------------------------------------------------------
def pooled_keep(b: Builder, x: Traced, qr: Traced, W: Callable[[str], Traced], p: str, positions: Traced,
                cached: Traced, ni: int, di: int, pool: int, pool_topk: int) -> Traced:
    """Additive mask ``[R, T, cap]`` of the pooled indexer (components/dsa.rs ``pooled_keep``).  ``cached[R, 1, cap,
    2 * di]`` holds every position's indexer key and pooling gate.  Every ``pool`` consecutive positions pool into one
    key - per channel, the keys weighted by the softmax over the pool's positions of ``gate + bias[position in pool]`` -
    and pool ``j`` is complete for a query at position ``q`` once ``(j + 1) * pool - 1 <= q``.  A query scores each
    complete pool ``sum_h w[h] / sqrt(ni) * relu(q_h . pooled) / sqrt(di)``, keeps the ``pool_topk`` best (equal scores:
    the lower pool) with all their positions, and every position after its last complete pool up to itself."""
    R, T = positions.shape
    cap = cached.shape[2]
    pools = cap // pool
    posf = b.cast(positions, F32)
    slots = b.cast(b.iota((R, T, cap), 2), F32)
    visible = b.binary("ge", b.broadcast(b.reshape(posf, (R, T, 1)), (R, T, cap)), slots)
    if pools == 0:
        keep = visible
    else:
        ends = b.cast(b.iota((R, T, pools), 2), F32) * float(pool) + float(pool - 1)
        complete = b.binary("ge", b.broadcast(b.reshape(posf, (R, T, 1)), (R, T, pools)), ends)          # [R, T, pools]
        tail_from = b.cast(complete, F32).sum(-1, keepdim=True) * float(pool)                             # [R, T, 1]
        block = b.reshape(b.slice(cached, 2, 0, pools * pool), (R, pools, pool, 2 * di))
        keys = b.slice(block, 3, 0, di)
        gates = b.slice(block, 3, di, di) + b.broadcast(b.reshape(W(p + "idx_pool_bias"), (1, 1, pool, di)), (R, pools, pool, di))
        wts = O.softmax(b, b.transpose(gates, (0, 1, 3, 2)))                                              # [R, pools, di, pool]
        pooled = (wts * b.transpose(keys, (0, 1, 3, 2))).sum(-1)                                          # [R, pools, di]
        q = b.transpose(b.reshape(O.linear(b, qr, W(p + "idx_q")), (R, T, ni, di)), (0, 2, 1, 3))         # [R, ni, T, di]
        pk = b.broadcast(b.reshape(b.transpose(pooled, (0, 2, 1)), (R, 1, di, pools)), (R, ni, di, pools))
        dots = O.relu(b, b.matmul(q, pk, "exact")) * (di ** -0.5)                                         # [R, ni, T, pools]
        hw = O.linear(b, x, W(p + "idx_weights"), precision="exact") * (ni ** -0.5)                       # [L, ni]
        hw = b.reshape(b.transpose(b.reshape(hw, (R, T, ni)), (0, 2, 1)), (R, ni, T, 1))
        score = (dots * b.broadcast(hw, dots.shape)).sum(1)                        # [R, T, pools]
        # incomplete pools rank after every complete one (they are the higher ids, so ties cannot lift them)
        score = b.select(complete, O.canonical_router_scores(b, score), b.broadcast(b.scalar(-O.F32_MAX, F32), score.shape))
        kept = min(pool_topk, pools)
        rank = b.reshape(O.stable_descending_rank(b, b.reshape(score, (R * T, pools))), (R, T, pools))
        chosen = b.binary("and", O.lnot(b, b.binary("ge", rank, b.broadcast(b.scalar(kept, I32), rank.shape))), complete)
        spread = b.reshape(b.broadcast(b.reshape(chosen, (R, T, pools, 1)), (R, T, pools, pool)), (R, T, pools * pool))
        tail = b.binary("and", b.binary("ge", slots, b.broadcast(tail_from, (R, T, cap))), visible)
        if pools * pool == cap:
            keep = b.binary("or", spread, tail)
        else:
            keep = b.concat([b.binary("or", spread, b.slice(tail, 2, 0, pools * pool)),
                             b.slice(tail, 2, pools * pool, cap - pools * pool)], 2)
    zero, hidden = b.scalar(0.0, F32), b.scalar(O.MASK_HIDDEN, F32)
    return b.select(keep, b.broadcast(zero, (R, T, cap)), b.broadcast(hidden, (R, T, cap)))


def pooled_dsa(b: Builder, x: Traced, W: Callable[[str], Traced], p: str, positions: Traced, read_map: Traced,
               write_map: Traced, slots: int, kv_dtype: DType, n_heads: int, qk: int, vd: int, rank: int, eps: float,
               ni: int, di: int, pool: int, pool_topk: int) -> Traced:
    """Latent attention without a rotary part whose queries read the positions a pooled indexer keeps
    (components/dsa.rs ``pooled_dsa``): low-rank query, the normalised latent cached per position (``c_pool``) and
    expanded through ``kv_b`` into every head's keys and values, the indexer's key and pooling gate cached beside it
    (``idx_pool``, ``2 * di`` wide), attention under :func:`pooled_keep`'s mask with scale ``qk ** -0.5``."""
    R, T = positions.shape
    L = R * T
    cap = read_map.shape[1]
    qr = O.rmsnorm(b, O.linear(b, x, W(p + "attn_q_a")), W(p + "attn_q_a_norm"), eps)
    q = b.transpose(b.reshape(O.linear(b, qr, W(p + "attn_q_b")), (R, T, n_heads, qk)), (0, 2, 1, 3))
    latent = O.rmsnorm(b, O.linear(b, x, W(p + "attn_kv_a")), W(p + "attn_kv_a_norm"), eps)

    def through_pool(name: str, rows_: Traced, width: int) -> Traced:
        pool_in = b.state(p + name, (slots, 1, width), kv_dtype, "blocked").cast(F32)
        nxt = b.scatter_update(pool_in, write_map, b.reshape(rows_, (L, 1, width)))
        b.output(nxt.cast(kv_dtype), p + name + ".next", "state_next", p + name)
        return O.paged_view(b, nxt.cast(kv_dtype).cast(F32), read_map)                                  # [R, 1, cap, width]

    c = through_pool("c_pool", latent, rank)
    key = O.layernorm(b, O.linear(b, x, W(p + "idx_k")), W(p + "idx_k_norm"), W(p + "idx_k_norm_bias"), 1e-6)
    cached = through_pool("idx_pool", b.concat([key, O.linear(b, x, W(p + "idx_pool_gate"))], -1), 2 * di)
    kv = O.linear(b, b.reshape(c, (R * cap, rank)), W(p + "attn_kv_b"))
    kv = b.transpose(b.reshape(kv, (R, cap, n_heads, qk + vd)), (0, 2, 1, 3))
    mask = pooled_keep(b, x, qr, W, p, positions, cached, ni, di, pool, pool_topk)
    a = O.attention_masked(b, q, b.slice(kv, 3, 0, qk), b.slice(kv, 3, qk, vd), mask, qk ** -0.5, 1, 0.0)
    return O.linear(b, b.reshape(b.transpose(a, (0, 2, 1, 3)), (L, n_heads * vd)), W(p + "attn_o"))


# ---- interleaved rotary on the trailing channels -----------------------------------------------------------------------
def rotate_tail(b: Builder, x: Traced, cos: Traced, sin: Traced, rot: int, inverse: bool = False) -> Traced:
    """Rotate the trailing ``rot`` channels of ``x[R, heads, n, D]`` as INTERLEAVED pairs ``(x[2i], x[2i + 1])`` by the
    angles of ``cos`` / ``sin`` (``[R, n, rot]`` rows of the duplicated-halves tables: entry ``i`` of the first half is
    pair ``i``'s); the leading channels pass through.  ``inverse`` turns the other way, which undoes the rotation at
    the same positions (crates/poot-models/src/architectures/deepseek4/sliding.rs ``rotate_tail``)."""
    R, Hh, n, D = x.shape
    half = rot // 2
    tail = b.reshape(b.slice(x, 3, D - rot, rot), (R, Hh, n, half, 2))
    a, c_ = b.reshape(b.slice(tail, 4, 0, 1), (R, Hh, n, half)), b.reshape(b.slice(tail, 4, 1, 1), (R, Hh, n, half))
    co = b.broadcast(b.reshape(b.slice(cos, -1, 0, half), (R, 1, n, half)), a.shape)
    si = b.broadcast(b.reshape(b.slice(sin, -1, 0, half), (R, 1, n, half)), a.shape)
    if inverse:
        si = -si
    out = b.concat([b.reshape(a * co - c_ * si, (R, Hh, n, half, 1)), b.reshape(a * si + c_ * co, (R, Hh, n, half, 1))], 4)
    out = b.reshape(out, (R, Hh, n, rot))
    return b.concat([b.slice(x, 3, 0, D - rot), out], 3) if rot < D else out


def pairwise_rank(b: Builder, s: Traced) -> Traced:
    """``rank[..., i]`` = how many entries of the last axis are STRICTLY greater than entry ``i``: exact ties share a
    rank, so a cut at ``k`` may keep more than ``k`` (the attention-side selectors' rule, unlike the router's stable
    rank; crates/poot-models/src/components/sparse_top_k.rs)."""
    shape = tuple(s.shape)
    n = shape[-1]
    mine = b.broadcast(b.reshape(s, shape + (1,)), shape + (n,))
    other = b.broadcast(b.reshape(s, shape[:-1] + (1, n)), shape + (n,))
    return b.cast(O.lnot(b, b.binary("ge", mine, other)), I32).sum(-1)


def softmax_pool(b: Builder, kv: Traced, gate: Traced) -> Traced:
    """``[R, windows, positions, channels] -> [R, windows, channels]``: per channel, the softmax of ``gate`` over a
    window's positions weights its ``kv`` rows."""
    w = b.transpose(O.softmax(b, b.transpose(gate, (0, 1, 3, 2))), (0, 1, 3, 2))
    return (kv * w).sum(2)


def paged_cache(b: Builder, name: str, rows_: Traced, slots: int, kv_dtype: DType, write_map: Traced, read_map: Traced) -> Traced:
    """Write this step's rows ``[L, width]`` into the paged pool ``name`` (one head) and read the sequence's positions
    back in order, through the storage dtype: ``[R, 1, cap, width]``."""
    L, width = rows_.shape
    pool_in = b.state(name, (slots, 1, width), kv_dtype, "blocked").cast(F32)
    nxt = b.scatter_update(pool_in, write_map, b.reshape(rows_, (L, 1, width)))
    b.output(nxt.cast(kv_dtype), name + ".next", "state_next", name)
    return O.paged_view(b, nxt.cast(kv_dtype).cast(F32), read_map)
