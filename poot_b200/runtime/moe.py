"""Mixture-of-experts FFN on the device engine (Mixtral / Qwen3-MoE / OLMoE style routed experts).

Two regimes, both on the grouped swap-AB tcgen05 kernel over the stacked expert weights:

* few (token, slot) pairs (``T * k <= E``, e.g. batch-1 decode): one group per pair reads only the experts that
  were selected (the reference's indexed GEMV, crates/poot-kernelgen/src/contraction/indexed.rs:1-6);
* otherwise the rows are grouped by expert on the device (``moe_align``: block-aligned runs, one expert per row tile),
  gathered into that order, multiplied by two grouped GEMMs that walk the tiles (the swap-AB kernel for tiles of up to
  64 rows, the tiled tcgen05 kernel for tiles of 128), and scattered back with a sum over each token's slots - every
  expert multiplies its own rows only, so the FLOPs are the routed FLOPs at any token count (the reference's
  group_expert_rows pass and grouped indexed contraction, passes/group_expert_rows.rs:1-8, contraction/indexed.rs:1-6).

Expert parallelism (an expert shard per rank, attention tensor-parallel): activations are replicated after the
attention block's all-reduce, so "dispatch" is a selection, not a transfer - each rank groups only the rows routed to
its own experts (any number of local experts) and the ranks' partial sums meet in one all-reduce.  In decode-sized
steps with one expert per rank the gate-scaled down projection is written straight into every rank's inbox from the
GEMM epilogue (the combine is the one-shot all-reduce fused into the expert GEMM).
"""
from __future__ import annotations

import torch

from ..ops import cuda_ops as K
from ..ops import moe_ops as M


def _buffers(eng):
    if getattr(eng, "_moe_buf", None) is None:
        c, dev = eng.cfg, eng.device
        T, E, k = eng.max_tokens, c.n_experts, c.top_k
        e_local = next((L_.ex_wgu.shape[0] for L_ in eng.w.layers if L_.ex_wgu is not None), E)
        F, H = c.moe_ffn, c.hidden
        any_packed = any(getattr(L_, "ex_packed", None) is not None for L_ in eng.w.layers)
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
            # experts kept packed run one activation row per (token, slot) at every step size
            "pact": torch.zeros(T * k, F, dtype=torch.bfloat16, device=dev) if any_packed else None,
            "pparts": torch.zeros(T * k, H, dtype=torch.bfloat16, device=dev) if any_packed else None,
        }
    return eng._moe_buf


def enable_expert_pool(eng, slots: int, manager) -> None:
    """Keep only ``slots`` experts of every routed layer on the device.  The stored expert tables move to pinned host
    memory, the device holds a pool ``[slots, ...]`` per table and an ``[E]`` map from expert id to pool row; each routed
    layer is cut at its router: the host reads the step's expert ids, ``manager.sync`` (an LRU residency manager: the
    driver's ``ExpertResidency``) names the rows to refill, the experts' bytes are copied as stored, and the layer runs
    its row-grouped program over the pool through the map.  Steps are launched eagerly (the cut is a host
    synchronisation, which a captured graph cannot hold).  The reference's pool transform and residency manager:
    crates/poot-graph-plan/src/passes/pool.rs:1-7, crates/poot-llm/src/driver/expert_residency.rs:1-14."""
    c = eng.cfg
    if not c.is_moe:
        raise ValueError("an expert pool needs routed experts")
    if c.expert_bias or eng.comm is not None:
        raise ValueError("the expert pool is built for unbiased experts on the single-device engine")
    if not (c.top_k <= slots < c.n_experts):
        raise ValueError(f"a pool of {slots} rows must hold a token's {c.top_k} experts and be smaller than the {c.n_experts} experts")
    pin = eng.device.type == "cuda"
    for L in eng.w.layers:
        if L.ex_wgu is None:
            continue
        host = (L.ex_wgu.cpu(), L.ex_wdown.cpu())
        L.ex_host = tuple(t.pin_memory() if pin else t for t in host)
        L.ex_wgu = torch.zeros(slots, *L.ex_wgu.shape[1:], dtype=L.ex_wgu.dtype, device=eng.device)
        L.ex_wdown = torch.zeros(slots, *L.ex_wdown.shape[1:], dtype=L.ex_wdown.dtype, device=eng.device)
        L.ex_map = torch.full((c.n_experts,), -1, dtype=torch.int32, device=eng.device)
    eng.expert_pool = (slots, manager)
    eng.use_graphs = False
    eng._moe_buf = None


def _pool_sync(eng, l: int, L, ids: torch.Tensor) -> torch.Tensor:
    """The host sync of a pooled routed layer: make the step's experts resident, return the ids as pool rows."""
    slots, mgr = eng.expert_pool
    E = eng.cfg.n_experts
    nbytes = sum(t[0].numel() * t[0].element_size() for t in L.ex_host)
    fills, emap, changed = mgr.sync((id(eng), l), ids.cpu().tolist(), E, slots, nbytes)
    for row, ex in fills:                                   # the stored bytes of each missing expert, as stored
        L.ex_wgu[row].copy_(L.ex_host[0][ex], non_blocking=True)
        L.ex_wdown[row].copy_(L.ex_host[1][ex], non_blocking=True)
    if changed:
        L.ex_map.copy_(torch.tensor(emap, dtype=torch.int32))
    return L.ex_map[ids.long()].contiguous()


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
        K.sigmoid_gate_rows_(act, g)
    h = eng.h[:T] if h is None else h
    K.linear(act, L.sh_wdown, K.EPI_RESID, h, h)


def _expert_act(eng, L, gu: torch.Tensor, act: torch.Tensor, idx: torch.Tensor, div: int, e0: int) -> None:
    """Bias of each row's expert (``idx[row // div] + e0``, when the family has one) and the gated activation over the
    (gate, up) pairs."""
    c = eng.cfg
    if L.ex_bgu is not None:
        eng._count()
        K.bias_add_indexed_(gu, L.ex_bgu, idx, div, e0)
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
    packed = getattr(L, "ex_packed", None)
    if packed is not None and (ep is not None or getattr(eng, "expert_pool", None) is not None):
        raise RuntimeError("experts kept packed run on one device without an expert pool")
    e_local = L.ex_wgu.shape[0] if packed is None else E
    e0 = eng.w.ep_rank * e_local
    logits = buf["logits"][:T]
    eng._count(2)
    if T > 128 and E % 8:        # the tiled GEMM wants 8-aligned N: narrow routers go through the skinny kernel in row chunks
        for t0 in range(0, T, 128):
            K.linear(x[t0:t0 + 128], L.router, K.EPI_F32, logits[t0:t0 + 128])
    else:
        K.linear(x, L.router, K.EPI_F32, logits)
    if L.router_bias is not None:
        K.bias_add_(logits, L.router_bias)
    ids, gates = buf["ids"][:T * k], buf["gates"][:T * k]
    dense = buf["dense"][:E * T].view(E, T)
    M.moe_route(logits, k, c.norm_topk_prob, ids, gates, dense, mode=c.router, select_bias=L.select_bias,
                scale=c.routed_scale, n_group=c.n_group, topk_group=c.topk_group)
    h = eng.h[:T] if h is None else h
    tp = (ep[1], ep[2]) if (ep is not None and ep[0] == "fused") else None
    pooled = getattr(eng, "expert_pool", None) is not None
    if pooled:
        eng._count()
        ids = _pool_sync(eng, l, L, ids)                    # expert ids -> pool rows; the layer below reads the pool
    if packed is not None:
        # the experts are read as stored: group g = (token, slot) multiplies the token's row with its expert's packed
        # gate and up rows (bias and gated activation fused), then with the packed down rows scaled by the slot's gate
        G = T * k
        act, parts = buf["pact"][:G], buf["pparts"][:G]
        eng._count(3)
        K.planar_gemv_grouped(x, packed, "in", ids, act, G, x_row_div=k, limit=c.swiglu_limit, alpha=c.swiglu_alpha)
        K.planar_gemv_grouped(act, packed, "out", ids, parts, G, row_scale=gates)
        M.moe_combine(h, parts, h, T, H, G, H, per_token=k)
        return None
    if ep is None and e_local == E and T * k <= E and not pooled:
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
            _expert_act(eng, L, gu, act, ids, 1, 0)
        M.gemm_grouped(K.EPI_STORE, act, L.ex_wdown, parts, 1, G, group_expert=ids, x_row_mul=1, out_group_stride=H,
                       row_scale=gates, ldo=H)
        if L.ex_bdown is not None:
            eng._count()
            K.bias_add_indexed_(parts, L.ex_bdown, ids, 1, 0, gate=gates)
        M.moe_combine(h, parts, h, T, H, G, H, per_token=k)
        return None
    if tp is not None and e_local == 1 and T <= 128:
        # decode-sized step with one expert per rank: the expert runs the step's rows with its gate column as the row
        # scale and its epilogue pushes the result into every rank's inbox (the combine is the fused all-reduce)
        act = buf["act"][:T * F].view(T, F)
        scale = dense[e0:e0 + 1, :T].contiguous()
        eng._count(2)
        M.gemm_grouped(K.EPI_SWIGLU, x, L.ex_wgu, act, T, 1, out_group_stride=T * F, ldo=F)
        M.gemm_grouped(K.EPI_STORE, act, L.ex_wdown, None, T, 1, x_row_mul=T, row_scale=scale, ldo=H, tp=tp)
        return "pushed"
    # Row-grouped regime: the (token, slot) rows of every local expert are made contiguous and padded to whole row
    # tiles (moe_align), the activations are gathered into that order, and two grouped GEMMs walk the tiles - each
    # expert multiplies its own rows only, at any token count and for any number of local experts.
    n = T * k
    block = M.group_block(n, E)
    max_tiles = M.group_capacity(n, e_local, block)
    cap = max_tiles * block
    g = _group_buffers(eng, cap, max_tiles, n)
    pos, sorted_rows, tile_expert, n_tiles = g["pos"][:n], g["sorted_rows"][:cap], g["tile_expert"][:max_tiles], g["n_tiles"]
    xs, gate_s = g["xs"][:cap], g["gate"][:cap]
    act, y = g["act"][:cap], g["y"][:cap]
    eng._count(4)
    M.moe_align(ids, e0, e_local, block, max_tiles, pos, sorted_rows, tile_expert, n_tiles)
    M.moe_gather_rows(x, sorted_rows, gates, n_tiles, block, max_tiles, k, xs, gate_s)
    plain = buf["gu"] is None
    tiled = block == 128 and L.ex_wgu.shape[1] % 128 == 0 and H % 128 == 0
    W2 = L.ex_wgu.shape[1]
    if plain:
        up_out, up_epi = act, K.EPI_SWIGLU
    else:               # biased / clamped / non-SwiGLU experts: plain projection, the tile's expert bias, then the activation
        up_out, up_epi = g["gu"][:cap], K.EPI_STORE
    if tiled:
        M.gemm_grouped_tiled(up_epi, xs, L.ex_wgu, up_out, tile_expert)
    else:
        M.gemm_grouped(up_epi, xs, L.ex_wgu, up_out, block, max_tiles, group_expert=tile_expert, x_row_mul=block,
                       out_group_stride=block * up_out.shape[1], ldo=up_out.shape[1])
    if not plain:
        _expert_act(eng, L, up_out, act, tile_expert, block, e0)
    if tiled:
        M.gemm_grouped_tiled(K.EPI_STORE, act, L.ex_wdown, y, tile_expert, row_scale=gate_s)
    else:
        M.gemm_grouped(K.EPI_STORE, act, L.ex_wdown, y, block, max_tiles, group_expert=tile_expert, x_row_mul=block,
                       out_group_stride=block * H, row_scale=gate_s, ldo=H)
    if L.ex_bdown is not None:      # the bias is part of the expert's output, so it is scaled by the row's gate too
        eng._count()
        K.bias_add_indexed_(y, L.ex_bdown, tile_expert, block, e0, gate=gate_s)
    eng._count()
    if ep is None:
        M.moe_scatter_combine(h, y, pos, h, T, H, k)
        return None
    if tp is not None:
        # any number of experts per rank, decode-sized step: the combine writes this rank's share of every token into
        # every rank's inbox (no library collective in the step)
        M.moe_scatter_combine_push(y, pos, T, H, k, tp)
        return "pushed"
    # expert parallel over the library collectives: this rank's experts' share of every token, summed over the ranks
    import torch.distributed as dist
    p = eng.comm.partial[:T]
    M.moe_scatter_combine(None, y, pos, p, T, H, k)
    dist.all_reduce(p, group=eng.comm.group)
    eng._count()
    K.add(h, p, out=h)
    return None


def moe_forward_sharded(eng, l: int, L, x: torch.Tensor, S: int, comm, site: int) -> None:
    """Routed experts over a token-sharded residual stream (the reduce-scatter form of tensor parallelism with the experts
    split over the same ranks): ``x[S, H]`` are THIS rank's normalised rows.  Router and top-k run on them; every
    (token, slot) row is dispatched to the rank that holds its expert; that rank groups what it received by expert, runs
    the two grouped GEMMs and sends each result row back; the owner adds its tokens' ``k`` rows to its residual shard
    (``comm.h_shard``).  Dispatch and combine are the all-to-all exchanges of ``csrc/kernels/ep_exchange.cu``."""
    c = eng.cfg
    E, k, F, H = c.n_experts, c.top_k, c.moe_ffn, c.hidden
    buf = _buffers(eng)
    e_local = L.ex_wgu.shape[0]
    e0 = eng.w.ep_rank * e_local
    logits = buf["logits"][:S]
    eng._count(2)
    K.linear(x, L.router, K.EPI_F32, logits)
    if L.router_bias is not None:
        eng._count()
        K.bias_add_(logits, L.router_bias)
    ids, gates = buf["ids"][:S * k], buf["gates"][:S * k]
    dense = buf["dense"][:E * S].view(E, S)
    M.moe_route(logits, k, c.norm_topk_prob, ids, gates, dense, mode=c.router, select_bias=L.select_bias,
                scale=c.routed_scale, n_group=c.n_group, topk_group=c.topk_group)
    eng._count(3)
    comm.ep_dispatch(x, ids, gates, S, k, e_local, site)                 # plan + peer stores + flags
    rids, _ = comm.ep_mask(S, k, e_local, site)                          # waits for every rank's rows
    n = comm.world * comm.ep_cap
    block = M.group_block(comm.world * S * k // comm.world, e_local)     # a rank receives S * k rows on average
    max_tiles = M.group_capacity(n, e_local, block)
    cap = max_tiles * block
    g = _group_buffers(eng, cap, max_tiles, n)
    pos, sorted_rows, tile_expert, n_tiles = g["pos"][:n], g["sorted_rows"][:cap], g["tile_expert"][:max_tiles], g["n_tiles"]
    xs, gate_s, act, y = g["xs"][:cap], g["gate"][:cap], g["act"][:cap], g["y"][:cap]
    eng._count(6)
    M.moe_align(rids, e0, e_local, block, max_tiles, pos, sorted_rows, tile_expert, n_tiles)
    comm.ep_gather(sorted_rows, n_tiles, block, max_tiles, xs, gate_s, S, k, e_local, site)
    plain = buf["gu"] is None
    up_out, up_epi = (act, K.EPI_SWIGLU) if plain else (g["gu"][:cap], K.EPI_STORE)
    M.gemm_grouped(up_epi, xs, L.ex_wgu, up_out, block, max_tiles, group_expert=tile_expert, x_row_mul=block,
                   out_group_stride=block * up_out.shape[1], ldo=up_out.shape[1])
    if not plain:
        _expert_act(eng, L, up_out, act, tile_expert, block, e0)
    M.gemm_grouped(K.EPI_STORE, act, L.ex_wdown, y, block, max_tiles, group_expert=tile_expert, x_row_mul=block,
                   out_group_stride=block * H, row_scale=gate_s, ldo=H)
    if L.ex_bdown is not None:
        eng._count()
        K.bias_add_indexed_(y, L.ex_bdown, tile_expert, block, e0, gate=gate_s)
    comm.ep_combine(y, pos, S, k, e_local, site)                         # peer stores + flags
    comm.ep_finish(S, k, e_local, site)                                  # waits, then h_shard += the tokens' k rows


def _group_buffers(eng, cap: int, max_tiles: int, n: int):
    """Scratch of the row-grouped regime, grown to the largest step seen (steps are captured per shape, so a buffer
    that a captured graph uses is never replaced: growth only happens before the first capture of a larger shape)."""
    c, dev = eng.cfg, eng.device
    g = getattr(eng, "_moe_group", None)
    if g is None or g["cap"] < cap or g["tiles"] < max_tiles or g["n"] < n:
        F, H = c.moe_ffn, c.hidden
        W2 = next(L_.ex_wgu.shape[1] for L_ in eng.w.layers if L_.ex_wgu is not None)
        need_gu = c.expert_bias or c.swiglu_limit > 0 or c.act != "silu" or not c.gated_ffn
        g = {"cap": cap, "tiles": max_tiles, "n": n,
             "pos": torch.zeros(n, dtype=torch.int32, device=dev),
             "sorted_rows": torch.zeros(cap, dtype=torch.int32, device=dev),
             "tile_expert": torch.zeros(max_tiles, dtype=torch.int32, device=dev),
             "n_tiles": torch.zeros(1, dtype=torch.int32, device=dev),
             "xs": torch.zeros(cap, H, dtype=torch.bfloat16, device=dev),
             "gate": torch.zeros(cap, dtype=torch.float32, device=dev),
             "act": torch.zeros(cap, F, dtype=torch.bfloat16, device=dev),
             "gu": torch.zeros(cap, W2, dtype=torch.bfloat16, device=dev) if need_gu else None,
             "y": torch.zeros(cap, H, dtype=torch.bfloat16, device=dev)}
        eng._moe_group = g
    return g
