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
