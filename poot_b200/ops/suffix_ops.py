"""Sampler-suffix device ops: sparse logit adjustment (+ guided mask) and the picked token's log-probability."""
from __future__ import annotations

from ctypes import c_int, c_void_p
from typing import Optional

import torch

from . import cuda_ops as K
from ._lib import check

_P = c_void_p
K.register_signature("poot_adjust_logits", [_P, c_int, c_int, _P, _P, c_int, _P, _P])
K.register_signature("poot_token_logprob", [_P, c_int, c_int, _P, _P, _P])


def adjust_logits(logits: torch.Tensor, idx: torch.Tensor, val: torch.Tensor, guided: Optional[torch.Tensor] = None) -> None:
    """In place: ``idx[rows, A]`` token ids (-1 = unused), ``val[rows, A, 4] = (bias, mul_pos, mul_neg, add)``."""
    rows, vocab = logits.shape
    check(K.fn("poot_adjust_logits")(logits.data_ptr(), rows, vocab, idx.data_ptr(), val.data_ptr(), idx.shape[1],
                                     None if guided is None else guided.data_ptr(), K._stream()), "adjust_logits")


def token_logprob(logits: torch.Tensor, picked: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=logits.device)
    check(K.fn("poot_token_logprob")(logits.data_ptr(), rows, vocab, picked.data_ptr(), out.data_ptr(), K._stream()),
          "token_logprob")
    return out
