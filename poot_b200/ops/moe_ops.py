"""Mixture-of-experts device ops: router top-k, grouped expert GEMM (swap-AB tcgen05 kernel over a stacked weight),
combine."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import cuda_ops as K
from ._lib import check

_P = c_void_p
K.register_signature("poot_moe_route", [_P, c_int, c_int, c_int, c_int, _P, _P, _P, _P])
K.register_signature("poot_moe_route_ex", [_P, c_int, c_int, c_int, c_int, c_int, _P, c_float, c_int, c_int, _P, _P, _P, _P])
K.register_signature("poot_moe_combine", [_P, _P, _P, c_int, c_int, c_int, c_longlong, c_int, _P])
K.register_signature("poot_gemm_skinny_grouped",
                     [c_int, _P, c_int, c_int, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int,
                      c_int, c_int, c_longlong, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, _P])


K.register_signature("poot_moe_align", [_P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P])
K.register_signature("poot_moe_gather_rows", [_P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, _P])
K.register_signature("poot_moe_scatter_combine", [_P, _P, _P, _P, c_int, c_int, c_int, _P])
K.register_signature("poot_gemm_grouped_tiled", [c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P])


def group_block(rows: int, experts: int) -> int:
    """Row tile of the grouped form for ``rows`` routed (token, slot) rows over ``experts`` experts: the smallest MMA
    token width that holds an average expert's rows, so padding stays below one tile per expert."""
    avg = max(1, rows // max(experts, 1))
    for b in (16, 32, 64):
        if avg <= b:
            return b
    return 128


def group_capacity(rows: int, experts: int, block: int) -> int:
    """Upper bound on row tiles: every expert's run is padded to a whole tile."""
    return (rows + block - 1) // block + experts


def moe_align(ids: torch.Tensor, e0: int, e_local: int, block: int, max_tiles: int, pos: torch.Tensor,
              sorted_rows: torch.Tensor, tile_expert: torch.Tensor, n_tiles: torch.Tensor) -> None:
    """Group the flat (token, slot) rows ``ids[n]`` by expert over this rank's experts ``[e0, e0 + e_local)``: ``pos[n]``
    (grouped position or -1), ``sorted_rows[max_tiles * block]`` (flat row or -1), ``tile_expert[max_tiles]`` (local expert
    of each tile or -1), ``n_tiles[1]``."""
    check(K.fn("poot_moe_align")(ids.data_ptr(), ids.numel(), e0, e_local, block, max_tiles, pos.data_ptr(),
                                 sorted_rows.data_ptr(), tile_expert.data_ptr(), n_tiles.data_ptr(), K._stream()), "moe_align")


def moe_gather_rows(x: torch.Tensor, sorted_rows: torch.Tensor, gates: torch.Tensor, n_tiles: torch.Tensor, block: int,
                    max_tiles: int, k: int, xs: torch.Tensor, gate_sorted: torch.Tensor) -> None:
    """``xs[p] = x[sorted_rows[p] // k]`` and ``gate_sorted[p] = gates[sorted_rows[p]]`` (zeros on padding rows)."""
    check(K.fn("poot_moe_gather_rows")(x.data_ptr(), x.stride(0), sorted_rows.data_ptr(), gates.data_ptr(), n_tiles.data_ptr(),
                                       block, max_tiles, k, x.shape[1], xs.data_ptr(), gate_sorted.data_ptr(), K._stream()),
          "moe_gather_rows")


def moe_scatter_combine(h: Optional[torch.Tensor], y: torch.Tensor, pos: torch.Tensor, out: torch.Tensor, T: int, H: int,
                        k: int) -> None:
    """``out[t] = (h[t] or 0) + sum_j y[pos[t * k + j]]`` over the slots with ``pos >= 0``."""
    check(K.fn("poot_moe_scatter_combine")(None if h is None else h.data_ptr(), y.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                           T, H, k, K._stream()), "moe_scatter_combine")


def gemm_grouped_tiled(epi: int, x: torch.Tensor, W: torch.Tensor, out: torch.Tensor, tile_expert: torch.Tensor,
                       row_scale: Optional[torch.Tensor] = None) -> None:
    """Tiled tcgen05 GEMM over rows grouped by expert in tiles of 128: ``x[M, K]`` with ``M = tiles * 128``, stacked
    ``W[E, N, K]``; tile ``t`` multiplies with expert ``tile_expert[t]`` (negative: unused)."""
    E, N, Kd = W.shape
    st = K.status_word(x.device)
    check(K.fn("poot_gemm_grouped_tiled")(epi, x.data_ptr(), W.data_ptr(), out.data_ptr(), x.shape[0], N, Kd, x.stride(0),
                                          out.stride(0), E, tile_expert.data_ptr(),
                                          None if row_scale is None else row_scale.data_ptr(), st.data_ptr(), K._stream()),
          "gemm_grouped_tiled")


def moe_route(logits: torch.Tensor, k: int, renorm: bool, ids: torch.Tensor, gates: torch.Tensor, dense: torch.Tensor,
              mode: str = "softmax", select_bias: Optional[torch.Tensor] = None, scale: float = 1.0, n_group: int = 1,
              topk_group: int = 1):
    """``logits[T,E]`` fp32 -> ``ids[T,k]`` i32, ``gates[T,k]`` f32, ``dense[E,T]`` f32 (0 where unselected).
    ``mode="sigmoid"``: per-expert sigmoid scores, ranked with ``select_bias[E]`` added (selection only), gates = the
    selected scores (over their sum when ``renorm``); every gate is multiplied by ``scale``."""
    T, E = logits.shape
    if mode == "softmax" and select_bias is None and scale == 1.0 and n_group == 1:
        check(K.fn("poot_moe_route")(logits.data_ptr(), T, E, k, int(renorm), ids.data_ptr(), gates.data_ptr(),
                                     dense.data_ptr(), K._stream()), "moe_route")
        return
    assert select_bias is None or (select_bias.dtype == torch.float32 and select_bias.numel() == E)
    check(K.fn("poot_moe_route_ex")(logits.data_ptr(), T, E, k, int(renorm), {"softmax": 0, "sigmoid": 1}[mode],
                                    None if select_bias is None else select_bias.data_ptr(), float(scale), int(n_group),
                                    int(topk_group), ids.data_ptr(),
                                    gates.data_ptr(), dense.data_ptr(), K._stream()), "moe_route_ex")


def moe_combine(h: Optional[torch.Tensor], parts: torch.Tensor, out: torch.Tensor, T: int, H: int, groups: int,
                gstride: int, per_token: int = 0) -> None:
    check(K.fn("poot_moe_combine")(None if h is None else h.data_ptr(), parts.data_ptr(), out.data_ptr(), T, H, groups,
                                   gstride, per_token, K._stream()), "moe_combine")


def moe_scatter_combine_push(y: torch.Tensor, pos: torch.Tensor, T: int, H: int, k: int, tp) -> None:
    """The expert-parallel combine of a decode-sized step fused with the one-shot all-reduce: this rank's share of every
    token goes straight into every rank's inbox; ``tp = (comm, rs_site)``.  The next reduce + norm kernel consumes it."""
    comm, rs_site = tp
    b = comm.block
    K.register_signature("poot_moe_scatter_combine_push", [_P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                           _P, _P, _P, _P, c_int, _P, _P, _P])
    check(K.fn("poot_moe_scatter_combine_push")(
        y.data_ptr(), pos.data_ptr(), T, H, k, comm.world, comm.rank, comm.MAX_ROWS, rs_site, comm.rs_sites,
        comm.epoch.data_ptr(), b.ptr(comm.rank, comm.off_flags), comm.flags_peer, comm.inbox_peer, comm.H,
        comm.ticket.data_ptr(), K.status_word(y.device).data_ptr(), K._stream()), "moe_scatter_combine_push")


def gemm_grouped(epi: int, x: torch.Tensor, W: torch.Tensor, out: Optional[torch.Tensor], M: int, groups: int,
                 group_expert: Optional[torch.Tensor] = None, x_row_div: int = 0, x_row_mul: int = 0,
                 x_col_per_expert: int = 0, out_group_stride: int = 0, row_scale: Optional[torch.Tensor] = None,
                 ldo: Optional[int] = None, K_dim: Optional[int] = None, tp=None) -> None:
    """Grouped skinny GEMM over stacked experts ``W[E, N, K]``; ``x`` is a 2-D activation buffer.

    ``tp = (comm, rs_site)`` sends the (single-group) result to every rank's inbox as a one-shot all-reduce
    contribution instead of writing ``out``."""
    E, N, Kw = W.shape
    Kd = K_dim or Kw
    ck = K.skinny_cluster(N, Kd)
    st = K.status_word(x.device)
    if ldo is None:
        ldo = out.stride(-2) if out is not None else N
    targs = (1, 0, 0, -1, 0, None, None, None, None, 0, None)
    if tp is not None:
        comm, rs_site = tp
        b = comm.block
        targs = (comm.world, comm.rank, comm.MAX_ROWS, rs_site, comm.rs_sites, comm.epoch.data_ptr(),
                 b.ptr(comm.rank, comm.off_flags), comm.flags_peer, comm.inbox_peer, comm.H, comm.ticket.data_ptr())
    check(K.fn("poot_gemm_skinny_grouped")(
        epi, x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), W.data_ptr(), E, None if out is None else out.data_ptr(),
        M, N, Kd, ldo, ck, groups, None if group_expert is None else group_expert.data_ptr(), x_row_div, x_row_mul,
        x_col_per_expert, out_group_stride, None if row_scale is None else row_scale.data_ptr(), st.data_ptr(),
        *targs, K._stream()), "gemm_skinny_grouped")
