"""Op library: every model-level operation as a composition of primitives.

These are the definitions the planner pattern-matches and the CPU oracle evaluates; device kernels are checked
against them.  Decompositions follow crates/poot-graph-ir/src/ops/*: ``rmsnorm`` (ops/norm.rs:4-29),
``layernorm`` (:32-75), ``linear`` (ops/linear.rs:8-19), half-split ``rope`` (ops/rope.rs:5-58), ``silu`` with a
single division and ``swiglu`` / ``gelu`` (ops/activation.rs:94-150), masked attention and ``paged_view``
(ops/attention.rs:7-337), causal masks from absolute positions (ops/prefill.rs), Mixtral-style routing
(ops/moe.rs:9-431) and the sampling suffix (ops/sampling.rs:277-440).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

from ..tensor import DType, alibi_slopes  # noqa: F401  (re-exported: callers take it from the op library)
from .builder import Builder, Traced

F32, I32 = DType.F32, DType.I32
MASK_HIDDEN = -1.0e9
F32_MAX = 3.4028234663852886e38


def lnot(b: Builder, x: Traced) -> Traced:
    """Logical not of a 0/1 I32 predicate (comparisons yield I32 0/1)."""
    return b.binary("xor", x, b.broadcast(b.scalar(1, I32), x.shape))


# ---- normalisation ---------------------------------------------------------------------------------------------
def rmsnorm(b: Builder, x: Traced, w: Traced, eps: float) -> Traced:
    D = x.shape[-1]
    sq = x * x
    ss = sq.sum(-1, keepdim=True)
    ms = ss * (1.0 / D)
    den = b.unary("sqrt", ms + eps)
    return (x / b.broadcast(den, x.shape)) * b.broadcast(w, x.shape)


def layernorm(b: Builder, x: Traced, w: Traced, bias: Optional[Traced], eps: float) -> Traced:
    D = x.shape[-1]
    mean = x.sum(-1, keepdim=True) * (1.0 / D)
    c = x - b.broadcast(mean, x.shape)
    var = (c * c).sum(-1, keepdim=True) * (1.0 / D)
    y = c / b.broadcast(b.unary("sqrt", var + eps), x.shape) * b.broadcast(w, x.shape)
    return y + b.broadcast(bias, x.shape) if bias is not None else y


def linear(b: Builder, x: Traced, w: Traced, bias: Optional[Traced] = None, precision: str = "narrow") -> Traced:
    """``x @ w^T`` for a checkpoint-order weight ``w[out, in]``."""
    y = b.matmul(x, b.transpose(w, (1, 0)), precision)
    return y + b.broadcast(bias, y.shape) if bias is not None else y


# ---- activations -----------------------------------------------------------------------------------------------
def sigmoid(b: Builder, x: Traced) -> Traced:
    return 1.0 / (1.0 + b.unary("exp", -x))


def silu(b: Builder, x: Traced) -> Traced:
    return x / (1.0 + b.unary("exp", -x))


def swiglu(b: Builder, gate: Traced, up: Traced) -> Traced:
    return silu(b, gate) * up


def relu(b: Builder, x: Traced) -> Traced:
    return b.binary("max", x, b.scalar(0.0, x.dtype))


def gelu_tanh(b: Builder, x: Traced) -> Traced:
    z = math.sqrt(2.0 / math.pi) * (x + 0.044715 * (x * x * x))
    return x / (1.0 + b.unary("exp", -2.0 * z))


def gelu_erf(b: Builder, x: Traced) -> Traced:
    return 0.5 * x * (1.0 + b.unary("erf", x * (1.0 / math.sqrt(2.0))))


def geglu(b: Builder, gate: Traced, up: Traced) -> Traced:
    return gelu_tanh(b, gate) * up


def softplus(b: Builder, x: Traced) -> Traced:
    return b.unary("log", 1.0 + b.unary("exp", x))


def softplus_stable(b: Builder, x: Traced) -> Traced:
    """``max(x, 0) + log(1 + exp(-|x|))``: softplus without overflow for large arguments."""
    zero = b.broadcast(b.scalar(0.0, F32), x.shape)
    ax = b.binary("max", x, -x)
    return b.binary("max", x, zero) + b.unary("log", 1.0 + b.unary("exp", -ax))


def l2norm(b: Builder, x: Traced, eps: float = 1e-6) -> Traced:
    return x / b.broadcast(b.unary("sqrt", (x * x).sum(-1, keepdim=True) + eps), x.shape)


def causal_conv1d(b: Builder, x: Traced, state: Traced, w: Traced, bias: Optional[Traced] = None):
    """Depthwise causal convolution of ``x[L, C]`` continuing from ``state[K-1, C]`` (the previous K-1 inputs) with
    taps ``w[C, K]``: ``y[t] = sum_k w[:, k] * xp[t + k]`` over ``xp = state ++ x``.  Returns ``(y, next_state)``
    (ops/ssm.rs causal conv1d)."""
    L, C = x.shape
    K = w.shape[1]
    xp = b.concat([state, x], 0)
    y = None
    for k in range(K):
        tap = b.broadcast(b.reshape(b.slice(w, 1, k, 1), (1, C)), (L, C))
        term = b.slice(xp, 0, k, L) * tap
        y = term if y is None else y + term
    if bias is not None:
        y = y + b.broadcast(bias, (L, C))
    return y, b.slice(xp, 0, L, K - 1)


def gated_rmsnorm(b: Builder, y: Traced, z: Traced, w: Traced, eps: float, gate_first: bool, gate_act: str = "silu") -> Traced:
    """RMSNorm over the last axis combined with a gate: ``norm(y * silu(z)) * w`` (Mamba2) or ``norm(y) * w * act(z)``
    (gated delta net; ``act`` is SiLU, or a sigmoid in Qwen3.8-Flash-Next)."""
    act = {"silu": silu, "sigmoid": sigmoid}[gate_act]
    if gate_first:
        return rmsnorm(b, y * act(b, z), w, eps)
    return rmsnorm(b, y, w, eps) * act(b, z)


def causal_conv1d_dilated(b: Builder, x: Traced, state: Traced, w: Traced, dilation: int):
    """Depthwise causal convolution whose taps are ``dilation`` positions apart: ``y[t] = sum_j w[:, j] *
    xp[t + j * dilation]`` over ``xp = state ++ x`` with ``state[(K - 1) * dilation, C]`` the previous inputs, oldest
    first.  Returns ``(y, next_state)`` (crates/poot-models/src/components/conv.rs)."""
    L, C = x.shape
    K = w.shape[1]
    xp = b.concat([state, x], 0)
    y = None
    for j in range(K):
        tap = b.broadcast(b.reshape(b.slice(w, 1, j, 1), (1, C)), (L, C))
        term = b.slice(xp, 0, j * dilation, L) * tap
        y = term if y is None else y + term
    return y, b.slice(xp, 0, L, (K - 1) * dilation)


def softcap(b: Builder, x: Traced, cap: float) -> Traced:
    return cap * b.unary("tanh", x * (1.0 / cap))


def softmax(b: Builder, x: Traced) -> Traced:
    m = x.max(-1, keepdim=True)
    e = b.unary("exp", x - b.broadcast(m, x.shape))
    return e / b.broadcast(e.sum(-1, keepdim=True), x.shape)


# ---- rotary ----------------------------------------------------------------------------------------------------
def rope(b: Builder, x: Traced, cos: Traced, sin: Traced, rot: Optional[int] = None) -> Traced:
    """Half-split rotary over the leading ``rot`` channels of ``x[..., heads, D]``; ``cos``/``sin`` are
    ``[tokens, rot]`` tables with duplicated halves, broadcast over heads."""
    D = x.shape[-1]
    rot = D if rot is None else rot
    half = rot // 2
    xr = b.slice(x, -1, 0, rot) if rot < D else x
    x1 = b.slice(xr, -1, 0, half)
    x2 = b.slice(xr, -1, half, half)
    rotated = b.concat([-x2, x1], -1)
    c = b.broadcast(b.reshape(cos, (cos.shape[0], 1, rot)), xr.shape)
    s = b.broadcast(b.reshape(sin, (sin.shape[0], 1, rot)), xr.shape)
    out = xr * c + rotated * s
    if rot < D:
        out = b.concat([out, b.slice(x, -1, rot, D - rot)], -1)
    return out


# ---- attention -------------------------------------------------------------------------------------------------
def repeat_kv(b: Builder, kv: Traced, n_rep: int) -> Traced:
    """Blocked GQA expansion ``[rows, kv_heads, S, D] -> [rows, kv_heads*n_rep, S, D]`` (q head h uses kv head h/n_rep)."""
    if n_rep == 1:
        return kv
    R, H, S, D = kv.shape
    x = b.broadcast(b.reshape(kv, (R, H, 1, S, D)), (R, H, n_rep, S, D))
    return b.reshape(x, (R, H * n_rep, S, D))


def causal_mask_from_pos(b: Builder, q_pos: Traced, cap: int, window: int = 0) -> Traced:
    """Additive mask ``[rows, tokens, cap]`` from absolute query positions ``[rows, tokens]``: key j is visible to a
    query at position p iff ``j <= p`` (and ``j > p - window`` with a sliding window)."""
    R, T = q_pos.shape
    keys = b.iota((R, T, cap), 2)
    p = b.broadcast(b.reshape(q_pos, (R, T, 1)), (R, T, cap))
    visible = b.binary("ge", p, keys)
    if window > 0:
        visible = b.binary("and", visible, b.binary("ge", keys, p - (window - 1)))
    zero, hidden = b.scalar(0.0, F32), b.scalar(MASK_HIDDEN, F32)
    return b.select(visible, b.broadcast(zero, (R, T, cap)), b.broadcast(hidden, (R, T, cap)))


def attention_masked(b: Builder, q: Traced, k: Traced, v: Traced, mask: Traced, scale: float, n_rep: int = 1,
                     cap: float = 0.0) -> Traced:
    """``softmax(q k^T * scale (+softcap) + mask) v`` with ``q[rows, heads, T, D]``, ``k/v[rows, kv_heads, S, D]`` and an
    additive ``mask[rows, T, S]``."""
    k, v = repeat_kv(b, k, n_rep), repeat_kv(b, v, n_rep)
    scores = b.matmul(q, b.transpose(k, (0, 1, 3, 2))) * scale
    if cap > 0:
        scores = softcap(b, scores, cap)
    R, H, T, S = scores.shape
    scores = scores + b.broadcast(b.reshape(mask, (R, 1, T, S)), scores.shape)
    return b.matmul(softmax(b, scores), v)


def alibi_bias_from_pos(b: Builder, q_pos: Traced, cap: int, slopes: Sequence[float]) -> Traced:
    """Per-head additive bias ``[rows, heads, tokens, cap]``: ``-slope[h] * (p - j)`` for a query at position p and key j
    (softmax is shift-invariant per row, so this equals the checkpoint families' ``slope * j`` forms)."""
    R, T = q_pos.shape
    keys = b.iota((R, T, cap), 2)
    p = b.broadcast(b.reshape(q_pos, (R, T, 1)), (R, T, cap))
    rel = b.reshape(b.cast(keys - p, F32), (R, 1, T, cap))
    return b.concat([rel * float(sl) for sl in slopes], 1)


def attention_biased(b: Builder, q: Traced, k: Traced, v: Traced, mask: Traced, scale: float, n_rep: int = 1,
                     cap: float = 0.0, head_bias: Optional[Traced] = None, sinks: Optional[Traced] = None) -> Traced:
    """:func:`attention_masked` plus a per-head additive bias ``[rows, heads, T, S]`` (ALiBi) and per-head sink logits
    ``[heads]`` that join every softmax denominator without contributing a value (ops/attention.rs ``attention_masked_sinks``)."""
    if head_bias is None and sinks is None:
        return attention_masked(b, q, k, v, mask, scale, n_rep, cap)
    k, v = repeat_kv(b, k, n_rep), repeat_kv(b, v, n_rep)
    scores = b.matmul(q, b.transpose(k, (0, 1, 3, 2))) * scale
    if cap > 0:
        scores = softcap(b, scores, cap)
    R, H, T, S = scores.shape
    if head_bias is not None:
        scores = scores + head_bias
    scores = scores + b.broadcast(b.reshape(mask, (R, 1, T, S)), scores.shape)
    if sinks is None:
        return b.matmul(softmax(b, scores), v)
    sk = b.broadcast(b.reshape(sinks, (1, H, 1, 1)), (R, H, T, 1))
    m = b.binary("max", scores.max(-1, keepdim=True), sk)
    e = b.unary("exp", scores - b.broadcast(m, scores.shape))
    den = e.sum(-1, keepdim=True) + b.unary("exp", sk - m)
    return b.matmul(e / b.broadcast(den, scores.shape), v)


def paged_view(b: Builder, pool: Traced, read_map: Traced) -> Traced:
    """Gather ``pool[slots, kv_heads, D]`` through ``read_map[rows, cap]`` into ``[rows, kv_heads, cap, D]``."""
    g = b.gather(pool, read_map, 0)                 # [rows, cap, kv_heads, D]
    return b.transpose(g, (0, 2, 1, 3))


# ---- mixture of experts ----------------------------------------------------------------------------------------
def canonical_router_scores(b: Builder, s: Traced) -> Traced:
    """NaN / -inf -> f32::MIN, +inf -> f32::MAX so ranks are total (``max`` is max-number: NaN is ignored)."""
    lo = b.broadcast(b.scalar(-F32_MAX, F32), s.shape)
    hi = b.broadcast(b.scalar(F32_MAX, F32), s.shape)
    return -b.binary("max", -b.binary("max", s, lo), -hi)


def stable_descending_rank(b: Builder, s: Traced) -> Traced:
    """``rank[r, e]`` = number of experts that sort before ``e`` (larger score, or equal score and lower index)."""
    R, E = s.shape
    a = b.broadcast(b.reshape(s, (R, E, 1)), (R, E, E))     # score of e
    o = b.broadcast(b.reshape(s, (R, 1, E)), (R, E, E))     # score of other f
    ie = b.iota((R, E, E), 1)
    io = b.iota((R, E, E), 2)
    gt = b.binary("ge", o, a)
    strictly = b.binary("and", gt, lnot(b, b.binary("ge", a, o)))               # o > a
    tie_before = b.binary("and", b.binary("and", gt, b.binary("ge", a, o)),      # o == a and f < e
                          lnot(b, b.binary("ge", io, ie)))
    before = b.binary("or", strictly, tie_before)
    return b.cast(before, I32).sum(-1)


def moe_topk_softmax(b: Builder, x: Traced, router: Traced, w_in: Traced, w_out: Traced, k: int,
                     precision: str = "narrow") -> Traced:
    """Mixtral routing: softmax over the selected top-k logits only; experts ``w_in[E, 2F, H]`` (gate rows then up
    rows), ``w_out[E, H, F]``; every token is evaluated by its k experts through ``indexed_matmul``."""
    L, H = x.shape
    E, F2, _ = w_in.shape
    F = F2 // 2
    scores = canonical_router_scores(b, linear(b, x, router, precision="exact"))
    rank = stable_descending_rank(b, scores)
    ids = b.arg_top_k(rank, k)                                              # [L, k]
    keep = lnot(b, b.binary("ge", rank, b.broadcast(b.scalar(k, I32), rank.shape)))
    neg = b.broadcast(b.scalar(MASK_HIDDEN, F32), scores.shape)
    sel = b.select(keep, scores, neg)
    m = sel.max(-1, keepdim=True)
    ex = b.unary("exp", sel - b.broadcast(m, sel.shape)) * b.cast(keep, F32)
    gates_all = ex / b.broadcast(ex.sum(-1, keepdim=True), ex.shape)        # [L, E]
    flat_ids = b.reshape(ids, (L * k,))
    gates = b.reshape(b.gather(b.reshape(gates_all, (L * E,)),
                               b.reshape(b.iota((L, k), 0) * E, (L * k,)) + flat_ids, 0), (L * k, 1))
    xr = b.reshape(b.broadcast(b.reshape(x, (L, 1, H)), (L, k, H)), (L * k, H))
    gu = b.indexed_matmul(xr, b.transpose(w_in, (0, 2, 1)), flat_ids, precision)     # [L*k, 2F]
    act = swiglu(b, b.slice(gu, -1, 0, F), b.slice(gu, -1, F, F))
    y = b.indexed_matmul(act, b.transpose(w_out, (0, 2, 1)), flat_ids, precision) * b.broadcast(gates, (L * k, H))
    return b.reshape(y, (L, k, H)).transpose(0, 2, 1).sum(-1)


def ffn_activation(b: Builder, gate: Traced, up: Optional[Traced], act: str = "silu", limit: float = 0.0,
                   alpha: float = 1.702) -> Traced:
    """``act(gate) * up`` for gated FFNs, ``act(gate)`` for plain ones.  ``limit > 0`` is the clamped form
    ``(min(up, limit) clamped below at -limit + 1) * g * sigmoid(alpha * g)`` with ``g = min(gate, limit)``."""
    if act == "silu_clamped":
        # silu(min(gate, limit)) * clamp(up, -limit, limit)   (components/ffn.rs ``Glu::ClampedSilu``)
        lim = b.broadcast(b.scalar(limit, F32), gate.shape)
        return swiglu(b, -b.binary("max", -gate, -lim), b.binary("max", -b.binary("max", -up, -lim), -lim))
    if limit > 0:
        lim = b.broadcast(b.scalar(limit, F32), gate.shape)
        g = -b.binary("max", -gate, -lim)
        u = b.binary("max", -b.binary("max", -up, -lim), -lim)
        return (u + 1.0) * (g / (1.0 + b.unary("exp", -(g * alpha))))
    a = {"silu": silu, "gelu_tanh": gelu_tanh, "gelu_erf": gelu_erf, "relu": relu,
         "relu2": lambda b_, x: relu(b_, x) * relu(b_, x)}[act](b, gate)
    return a * up if up is not None else a


def _top2_sum(b: Builder, s: Traced) -> Traced:
    """Sum of the two largest entries along the last axis (ties counted twice)."""
    m1 = s.max(-1, keepdim=True)
    is_max = b.binary("ge", s, b.broadcast(m1, s.shape))
    cnt = b.cast(is_max, I32).sum(-1, keepdim=True)
    rest = b.select(is_max, b.broadcast(b.scalar(-F32_MAX, F32), s.shape), s).max(-1, keepdim=True)
    two = b.binary("ge", cnt, b.broadcast(b.scalar(2, I32), cnt.shape))
    return b.reshape(m1 + b.select(two, m1, rest), s.shape[:-1])


def moe_routed(b: Builder, x: Traced, router: Traced, w_in: Traced, w_out: Traced, k: int, *,
               score: str = "softmax", renorm: bool = True, router_bias: Optional[Traced] = None,
               select_bias: Optional[Traced] = None, n_group: int = 1, topk_group: int = 1, routed_scale: float = 1.0,
               act: str = "silu", limit: float = 0.0, alpha: float = 1.702, in_bias: Optional[Traced] = None,
               out_bias: Optional[Traced] = None, gated: bool = True, precision: str = "narrow",
               router_x: Optional[Traced] = None, expert_scale: Optional[Traced] = None,
               route_ids: Optional[Traced] = None) -> Traced:
    """Routed experts in every variant the shipped families use (components/router.rs, ops/moe.rs).

    ``score``: ``softmax`` over all experts or ``sigmoid`` per expert.  Selection ranks ``score + select_bias`` (the
    bias does not enter the gate), optionally restricted to the ``topk_group`` best of ``n_group`` expert groups
    (group score = sum of its two best selection scores; experts outside are ranked as 0).  Gates are the scores at
    the selected experts, divided by their sum when ``renorm``, times ``routed_scale``.  Experts: ``w_in[E, 2F, H]``
    gate rows then up rows (+ ``in_bias[E, 2F]``), ``w_out[E, H, F]`` (+ ``out_bias[E, H]``); with ``gated=False``
    ``w_in[E, F, H]`` and the expert is ``down(act(up(x)))``.  ``router_x``: the router reads these rows instead of
    the experts' input; ``expert_scale[E]`` multiplies the gate of each expert after the renormalisation.
    ``score="sqrtsoftplus"``: ``sqrt(softplus(logit))`` per expert (DeepSeek-V4).  ``route_ids[L, k]`` I32: the experts
    come from a table instead of a ranking (a hash-routed layer); they are gated by their own scores, normalised over
    the selection when ``renorm``, times ``routed_scale`` (architectures/deepseek4/moe.rs ``hash_routes``)."""
    L, H = x.shape
    E, F2, _ = w_in.shape
    F = F2 // 2 if gated else F2
    logits = linear(b, router_x if router_x is not None else x, router, router_bias, precision="exact")
    scored = {"softmax": lambda t: softmax(b, t), "sigmoid": lambda t: sigmoid(b, t),
              "sqrtsoftplus": lambda t: b.unary("sqrt", softplus_stable(b, t))}[score]
    if route_ids is not None:
        probs = canonical_router_scores(b, scored(logits))
        flat_ids = b.reshape(route_ids, (L * k,))
        sel = b.reshape(b.gather(b.reshape(probs, (L * E,)), b.reshape(b.iota((L, k), 0) * E, (L * k,)) + flat_ids, 0), (L, k))
        if renorm:
            sel = sel / b.broadcast(sel.sum(-1, keepdim=True), sel.shape)
        gates = b.reshape(sel * routed_scale if routed_scale != 1.0 else sel, (L * k, 1))
        return _experts(b, x, w_in, w_out, flat_ids, gates, k, act, limit, alpha, in_bias, out_bias, gated, precision)
    if score == "softmax" and renorm and select_bias is None and n_group == 1:
        # softmax over all, pick k, renormalise == softmax over the k selected logits
        scores = canonical_router_scores(b, logits)
        rank = stable_descending_rank(b, scores)
        keep = lnot(b, b.binary("ge", rank, b.broadcast(b.scalar(k, I32), rank.shape)))
        sel = b.select(keep, scores, b.broadcast(b.scalar(MASK_HIDDEN, F32), scores.shape))
        m = sel.max(-1, keepdim=True)
        ex = b.unary("exp", sel - b.broadcast(m, sel.shape)) * b.cast(keep, F32)
        gates_all = ex / b.broadcast(ex.sum(-1, keepdim=True), ex.shape)
    else:
        probs = scored(logits)
        choice = probs + b.broadcast(select_bias, probs.shape) if select_bias is not None else probs
        choice = canonical_router_scores(b, choice)
        if n_group > 1:
            per = E // n_group
            gs = _top2_sum(b, b.reshape(choice, (L, n_group, per)))                  # [L, G]
            grank = stable_descending_rank(b, gs)
            gkeep = lnot(b, b.binary("ge", grank, b.broadcast(b.scalar(topk_group, I32), grank.shape)))
            ekeep = b.reshape(b.broadcast(b.reshape(gkeep, (L, n_group, 1)), (L, n_group, per)), (L, E))
            choice = b.select(ekeep, choice, b.broadcast(b.scalar(0.0, F32), choice.shape))
        rank = stable_descending_rank(b, choice)
        keep = b.cast(lnot(b, b.binary("ge", rank, b.broadcast(b.scalar(k, I32), rank.shape))), F32)
        picked = probs * keep
        if renorm:
            den = picked.sum(-1, keepdim=True)
            if score == "sigmoid":
                den = den + 1e-20
            picked = picked / b.broadcast(den, picked.shape)
        gates_all = picked * routed_scale if routed_scale != 1.0 else picked
    if expert_scale is not None:
        gates_all = gates_all * b.broadcast(b.reshape(expert_scale, (1, E)), gates_all.shape)
    ids = b.arg_top_k(rank, k)                                              # [L, k]
    flat_ids = b.reshape(ids, (L * k,))
    gates = b.reshape(b.gather(b.reshape(gates_all, (L * E,)),
                               b.reshape(b.iota((L, k), 0) * E, (L * k,)) + flat_ids, 0), (L * k, 1))
    return _experts(b, x, w_in, w_out, flat_ids, gates, k, act, limit, alpha, in_bias, out_bias, gated, precision)


def _experts(b: Builder, x: Traced, w_in: Traced, w_out: Traced, flat_ids: Traced, gates: Traced, k: int, act: str,
             limit: float, alpha: float, in_bias: Optional[Traced], out_bias: Optional[Traced], gated: bool,
             precision: str) -> Traced:
    """Every token through its ``k`` routed experts (``flat_ids[L * k]``, ``gates[L * k, 1]``) and their gated sum."""
    L, H = x.shape
    F2 = w_in.shape[1]
    F = F2 // 2 if gated else F2
    xr = b.reshape(b.broadcast(b.reshape(x, (L, 1, H)), (L, k, H)), (L * k, H))
    gu = b.indexed_matmul(xr, b.transpose(w_in, (0, 2, 1)), flat_ids, precision)     # [L*k, 2F]
    if in_bias is not None:
        gu = gu + b.gather(in_bias, flat_ids, 0)
    a = ffn_activation(b, b.slice(gu, -1, 0, F), b.slice(gu, -1, F, F), act, limit, alpha) if gated else \
        ffn_activation(b, gu, None, act)
    y = b.indexed_matmul(a, b.transpose(w_out, (0, 2, 1)), flat_ids, precision)
    if out_bias is not None:
        y = y + b.gather(out_bias, flat_ids, 0)
    y = y * b.broadcast(gates, (L * k, H))
    return b.reshape(y, (L, k, H)).transpose(0, 2, 1).sum(-1)


# ---- sampling suffix -------------------------------------------------------------------------------------------
def sample_head(b: Builder, logits: Traced, rule: str = "greedy", seed: Optional[Traced] = None,
                params: Optional[Traced] = None, top_k: Optional[Traced] = None, bias: Optional[Traced] = None,
                guided_mask: Optional[Traced] = None) -> Traced:
    """Adjusted logits (+bias, +guided mask) then ``sample_token``; Gumbel noise is ``-ln(-ln u)`` of the exact
    uniform draw.  Returns ``[rows, 2]`` I32 ``(token, non_finite_index)``."""
    if bias is not None:
        logits = logits + bias
    if guided_mask is not None:
        logits = logits + guided_mask
    if rule == "greedy":
        return b.sample_token("greedy", logits)
    u = b.random_uniform(seed, logits.shape[-1])
    noise = -b.unary("log", -b.unary("log", u))
    return b.sample_token(rule, logits, noise, params, top_k if rule != "gumbel" else None)


# ---- chunk-parallel gated delta rule ---------------------------------------------------------------------------------
def delta_rule_chunked(b: Builder, q: Traced, k: Traced, v: Traced, g: Traced, beta: Traced, s_in: Traced, chunk: int = 64):
    """The gated delta rule of the ``scan`` equation (one log decay per head and token) in its chunk-parallel form: the
    same ``(y[1, H, L, D], state[1, H, D, D])`` out of matrix products over chunks of ``chunk`` tokens instead of one step
    per token (crates/poot-graph-ir/src/ops/prefill.rs: the chunked linear-attention prefill).

    Within a chunk, with ``G`` the running sum of the log decays, ``M[i, j] = beta_i (k_i . k_j) exp(G_i - G_j)`` for
    ``j < i`` couples a token's correction to the earlier ones; ``T = (I + M)^-1`` undoes the coupling.  ``M`` is strictly
    lower triangular, so with ``X = -M`` the inverse is the finite product ``(I + X)(I + X^2)(I + X^4)...`` -
    ``log2(chunk)`` squarings, all matrix products.  Then per chunk, from the state ``S`` carried in:

        ``v' = T (beta v) - T (beta k exp(G)) S``
        ``y  = (q exp(G)) S + tril(q k^T exp(G_i - G_j)) v'``
        ``S  = exp(G_last) S + (k exp(G_last - G))^T v'``

    A ragged last chunk is padded with tokens that change nothing (zero key, value, beta and log decay)."""
    _, H, L, D = q.shape
    if tuple(g.shape) != (1, H, L, 1):
        raise ValueError("the chunk-parallel form needs one log decay per head and token")
    C = chunk
    n = -(-L // C)
    pad = n * C - L

    def chunks(t: Traced, width: int) -> Traced:                      # [1, H, L, width] -> [H, n, C, width]
        t = b.reshape(t, (H, L, width))
        if pad:
            t = b.concat([t, b.broadcast(b.scalar(0.0, F32), (H, pad, width))], 1)
        return b.reshape(t, (H, n, C, width))

    qc, kc, vc, gc, bc = chunks(q, D), chunks(k, D), chunks(v, D), chunks(g, 1), chunks(beta, 1)
    row, col = b.iota((H, n, C, C), 2), b.iota((H, n, C, C), 3)
    lower_incl = b.cast(b.binary("ge", row, col), F32)                 # j <= i
    strictly = lower_incl - b.cast(b.binary("ge", col, row), F32) * lower_incl          # j < i
    G = b.matmul(lower_incl, gc, "exact")                              # running sum of the log decays: [H, n, C, 1]
    Gt = b.transpose(G, (0, 1, 3, 2))
    # exp(G_i - G_j) only where j <= i (above the diagonal the difference is positive and may overflow)
    decay = b.unary("exp", (b.broadcast(G, (H, n, C, C)) - b.broadcast(Gt, (H, n, C, C))) * lower_incl) * lower_incl
    kb = kc * b.broadcast(bc, kc.shape)
    X = -(b.matmul(kb, b.transpose(kc, (0, 1, 3, 2)), "exact") * decay * strictly)
    eye = lower_incl * b.cast(b.binary("ge", col, row), F32)
    T, P, span = eye + X, X, 1
    while span * 2 < C:
        P = b.matmul(P, P, "exact")
        T = b.matmul(T, eye + P, "exact")
        span *= 2
    eG = b.unary("exp", G)
    value = b.matmul(T, vc * b.broadcast(bc, vc.shape), "exact")       # T (beta v)
    k_cum = b.matmul(T, kb * b.broadcast(eG, kb.shape), "exact")       # T (beta k exp(G))
    qk = b.matmul(qc, b.transpose(kc, (0, 1, 3, 2)), "exact") * decay  # tril(q k^T exp(G_i - G_j)), diagonal kept
    q_in = qc * b.broadcast(eG, qc.shape)
    G_last = b.slice(G, 2, C - 1, 1)                                   # [H, n, 1, 1]
    k_out = kc * b.broadcast(b.unary("exp", b.broadcast(G_last, G.shape) - G), kc.shape)
    e_last = b.unary("exp", G_last)
    S = b.reshape(s_in, (H, D, D))
    ys = []
    for c in range(n):
        pick = lambda t: b.reshape(b.slice(t, 1, c, 1), (H,) + tuple(t.shape[2:]))
        v_new = pick(value) - b.matmul(pick(k_cum), S, "exact")
        ys.append(b.matmul(pick(q_in), S, "exact") + b.matmul(pick(qk), v_new, "exact"))
        S = S * b.broadcast(pick(e_last), (H, D, D)) + b.matmul(b.transpose(pick(k_out), (0, 2, 1)), v_new, "exact")
    y = b.concat(ys, 1) if n > 1 else ys[0]
    if pad:
        y = b.slice(y, 1, 0, L)
    return b.reshape(y, (1, H, L, D)), b.reshape(S, (1, H, D, D))
