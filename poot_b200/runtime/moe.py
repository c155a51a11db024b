"""Mixture-of-experts FFN on the device engine (Mixtral / Qwen3-MoE / OLMoE style routed experts).

Two regimes, both on the grouped swap-AB tcgen05 kernel over the stacked expert weights:

* few (token, slot) pairs (``T * k <= E``, e.g. batch-1 decode): one group per pair reads only the experts that
  were selected (the reference's indexed GEMV, crates/poot-kernelgen/src/contraction/indexed.rs:1-6);
* otherwise: one group per expert runs all T tokens; the dense gate matrix (0 for an unselected expert) scales the
  rows of the down projection, and the combine kernel adds the E outputs to the residual stream - every expert
  weight is read exactly once per step (the reference groups rows by expert, passes/group_expert_rows.rs:1-8).

Expert parallelism (one expert shard per rank, attention tensor-parallel): activations are replicated after the
fused all-reduce, so no dispatch transfer is needed; each rank runs its local experts over all tokens and the
gate-scaled down projection is written straight into every rank's inbox - the combine all-to-all is the one-shot
all-reduce fused into the expert GEMM's epilogue.
"""
from __future__ import annotations

import torch

from ..ops import cuda_ops as K
from ..ops import moe_ops as M


def _buffers(eng):
    if getattr(eng, "_moe_buf", None) is None:
        c, dev = eng.cfg, eng.device
        T, E, k = eng.max_tokens, c.n_experts, c.top_k
        e_local = next(L_.ex_wgu.shape[0] for L_ in eng.w.layers if L_.ex_wgu is not None)
        F, H = c.moe_ffn, c.hidden
        Tc = min(T, 128)
        G = max(e_local, min(T, E) * k)
        eng._moe_buf = {
            "logits": torch.zeros(T, E, dtype=torch.float32, device=dev),
            "ids": torch.zeros(T * k, dtype=torch.int32, device=dev),
            "gates": torch.zeros(T * k, dtype=torch.float32, device=dev),
            "dense": torch.zeros(E * T, dtype=torch.float32, device=dev),
            "act": torch.zeros(G * Tc * F, dtype=torch.bfloat16, device=dev),
            "gu": (torch.zeros(G * Tc * 2 * F, dtype=torch.bfloat16, device=dev)
                   if (c.expert_bias or c.swiglu_limit > 0 or c.act != "silu" or not c.gated_ffn) else None),
            "parts": torch.zeros(G * Tc * H, dtype=torch.bfloat16, device=dev),
        }
    return eng._moe_buf


def shared_expert(eng, L, x: torch.Tensor, T: int, h=None) -> None:
    """``h[:T] += shared(x)``: the always-on expert of families that have one (a dense SwiGLU FFN), optionally scaled per
    token by ``sigmoid(x . w)`` (the scale is applied to the activation rows, which the down projection carries through)."""
    c = eng.cfg
    if getattr(eng, "_sh_act", None) is None:
        eng._sh_act = torch.zeros(eng.max_tokens, c.shared_width, dtype=torch.bfloat16, device=eng.device)
        eng._sh_gate = torch.zeros(eng.max_tokens, 8, dtype=torch.float32, device=eng.device)
    act = eng._sh_act[:T]
    eng._count(2)
    if c.gated_ffn:
        K.linear(x, L.sh_wgu, K.EPI_SWIGLU, act)
    else:
        eng._count()
        K.linear(x, L.sh_wgu, K.EPI_STORE, act)
        K.act_(act, c.act)
    if L.sh_gate is not None:
        eng._count(2)
        g = eng._sh_gate[:T]
        K.linear(x, L.sh_gate, K.EPI_F32, g)
        act.mul_(torch.sigmoid(g[:, :1]).to(act.dtype))
    h = eng.h[:T] if h is None else h
    K.linear(act, L.sh_wdown, K.EPI_RESID, h, h)


def _expert_act(eng, L, gu: torch.Tensor, act: torch.Tensor, expert_of_row: torch.Tensor) -> None:
    """Bias of each row's expert (when the family has one) and the gated activation over the (gate, up) pairs."""
    c = eng.cfg
    if L.ex_bgu is not None:
        gu.add_(L.ex_bgu[expert_of_row])
    eng._count()
    if not c.gated_ffn:                 # experts without a gate: act(up(x))
        act.copy_(gu)
        K.act_(act, c.act)
    elif c.swiglu_limit > 0:
        K.gated_act(gu, True, "swiglu_clamped", out=act, limit=c.swiglu_limit, alpha=c.swiglu_alpha)
    else:
        K.gated_act(gu, True, c.act, out=act)


def moe_forward(eng, l: int, L, x: torch.Tensor, T: int, ep=None, h=None):
    """``h[:T] += moe(x)``.  ``ep`` selects the expert-parallel form: ``("nccl", comm)`` reduces the local experts'
    partial with a library all-reduce, ``("fused", comm, rs_site)`` pushes it into every rank's inbox from the GEMM
    epilogue (returns ``"pushed"``: the caller's next reduce+norm kernel consumes it)."""
    c = eng.cfg
    E, k, F, H = c.n_experts, c.top_k, c.moe_ffn, c.hidden
    buf = _buffers(eng)
    e_local = L.ex_wgu.shape[0]
    e0 = eng.w.ep_rank * e_local
    logits = buf["logits"][:T]
    eng._count(2)
    if T > 128 and E % 8:        # the tiled GEMM wants 8-aligned N: narrow routers go through the skinny kernel in row chunks
        for t0 in range(0, T, 128):
            K.linear(x[t0:t0 + 128], L.router, K.EPI_F32, logits[t0:t0 + 128])
    else:
        K.linear(x, L.router, K.EPI_F32, logits)
    if L.router_bias is not None:
        logits.add_(L.router_bias)
    ids, gates = buf["ids"][:T * k], buf["gates"][:T * k]
    dense = buf["dense"][:E * T].view(E, T)
    M.moe_route(logits, k, c.norm_topk_prob, ids, gates, dense, mode=c.router, select_bias=L.select_bias,
                scale=c.routed_scale, n_group=c.n_group, topk_group=c.topk_group)
    h = eng.h[:T] if h is None else h
    tp = (ep[1], ep[2]) if (ep is not None and ep[0] == "fused") else None
    if ep is None and e_local == E and T * k <= E:
        G = T * k                                             # one group per (token, slot)
        act = buf["act"][:G * F].view(G, F)
        parts = buf["parts"][:G * H].view(G, H)
        eng._count(3)
        if buf["gu"] is None:
            M.gemm_grouped(K.EPI_SWIGLU, x, L.ex_wgu, act, 1, G, group_expert=ids, x_row_div=k, out_group_stride=F, ldo=F)
        else:           # biased / clamped experts: plain projection, bias of the group's expert, then the activation
            W2 = L.ex_wgu.shape[1]          # 2F with a gate, F without
            gu = buf["gu"][:G * W2].view(G, W2)
            M.gemm_grouped(K.EPI_STORE, x, L.ex_wgu, gu, 1, G, group_expert=ids, x_row_div=k, out_group_stride=W2, ldo=W2)
            _expert_act(eng, L, gu, act, ids.long())
        M.gemm_grouped(K.EPI_STORE, act, L.ex_wdown, parts, 1, G, group_expert=ids, x_row_mul=1, out_group_stride=H,
                       row_scale=gates, ldo=H)
        if L.ex_bdown is not None:
            parts.add_((L.ex_bdown[ids.long()].float() * gates[:, None]).to(parts.dtype))
        M.moe_combine(h, parts, h, T, H, G, H, per_token=k)
        return None
    if ep is not None and e_local == 1 and T > 128:
        # prefill with one expert per rank: two tiled GEMMs over all T rows (the expert's weights are read once);
        # the gate (0 for tokens routed elsewhere) scales the activation rows before the down projection
        act = eng.act[:T]
        eng._count(4)
        K.linear(x, L.ex_wgu[0], K.EPI_SWIGLU, act)
        act.mul_(dense[e0, :T].unsqueeze(1))
        import torch.distributed as dist
        p = eng.comm.partial[:T]
        K.linear(act, L.ex_wdown[0], K.EPI_STORE, p)
        dist.all_reduce(p, group=eng.comm.group)
        K.add(h, p, out=h)
        return None
    # dense-over-experts regime, in token chunks of at most 128 rows
    for t0 in range(0, T, 128):
        n = min(128, T - t0)
        xs = x[t0:t0 + n]
        act = buf["act"][:e_local * n * F].view(e_local * n, F)
        scale = dense[e0:e0 + e_local, t0:t0 + n].contiguous() if (t0 or n != T or e_local != E) else dense
        eng._count(2)
        if buf["gu"] is None:
            M.gemm_grouped(K.EPI_SWIGLU, xs, L.ex_wgu, act, n, e_local, out_group_stride=n * F, ldo=F)
        else:
            W2 = L.ex_wgu.shape[1]
            gu = buf["gu"][:e_local * n * W2].view(e_local * n, W2)
            M.gemm_grouped(K.EPI_STORE, xs, L.ex_wgu, gu, n, e_local, out_group_stride=n * W2, ldo=W2)
            _expert_act(eng, L, gu, act, torch.arange(e0, e0 + e_local, device=gu.device).repeat_interleave(n))
        if tp is not None and e_local == 1 and T <= 128:
            M.gemm_grouped(K.EPI_STORE, act, L.ex_wdown, None, n, 1, x_row_mul=n, row_scale=scale, ldo=H, tp=tp)
            return "pushed"
        parts = buf["parts"][:e_local * n * H].view(e_local * n, H)
        M.gemm_grouped(K.EPI_STORE, act, L.ex_wdown, parts, n, e_local, x_row_mul=n, out_group_stride=n * H,
                       row_scale=scale, ldo=H)
        if L.ex_bdown is not None:      # the bias is part of the expert's output, so it is scaled by the row's gate too
            sc = dense[e0:e0 + e_local, t0:t0 + n].reshape(e_local * n, 1)
            parts.add_((L.ex_bdown[e0:e0 + e_local].float().repeat_interleave(n, 0) * sc).to(parts.dtype))
        eng._count()
        if ep is None:
            M.moe_combine(h[t0:t0 + n], parts, h[t0:t0 + n], n, H, e_local, n * H)
        else:
            M.moe_combine(None, parts, eng.comm.partial[t0:t0 + n], n, H, e_local, n * H)
    if ep is not None:      # library all-reduce over the ranks' expert partials, then the residual add
        import torch.distributed as dist
        p = eng.comm.partial[:T]
        dist.all_reduce(p, group=eng.comm.group)
        eng._count()
        K.add(h, p, out=h)
    return None
