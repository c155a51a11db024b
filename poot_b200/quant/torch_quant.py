"""Whole-tensor Q4_K and Q8_0 encoders written with torch ops, so they run where the tensor lives.

They make the same choices as the host codec's encoders (min/max sub-block ranges, 6-bit scale/min codes against an
fp16 super-block scale, round-to-nearest levels; layouts of ggml's ``block_q4_K`` / ``block_q8_0`` as the reference
decodes them, crates/poot-quant/src/blocks.rs:174-192 and :293-346) and exist so an 8-billion-parameter random
model can be quantised on the device in seconds instead of on the host in minutes.
"""
from __future__ import annotations

import torch


def _round_half_away(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.floor(torch.abs(x) + 0.5)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    """``[rows, cols]`` float -> ``[rows, cols/32 * 34]`` uint8 (fp16 scale then 32 int8 levels per block)."""
    rows, cols = w.shape
    assert cols % 32 == 0
    x = w.float().reshape(rows, cols // 32, 32)
    amax = x.abs().amax(dim=-1, keepdim=True)
    d = (amax / 127.0).to(torch.float16)
    df = d.float()
    inv = torch.where(df > 0, 1.0 / df, torch.zeros_like(df))
    q = _round_half_away(x * inv).clamp_(-127, 127).to(torch.int8)
    out = torch.empty(rows, cols // 32, 34, dtype=torch.uint8, device=w.device)
    out[..., :2] = d.view(torch.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = q.view(torch.uint8)
    return out.reshape(rows, -1)


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """``[rows, cols]`` float -> ``[rows, cols/256 * 144]`` uint8 (d, dmin fp16 | 12 scale bytes | 128 nibble bytes)."""
    rows, cols = w.shape
    assert cols % 256 == 0
    nb = cols // 256
    x = w.float().reshape(rows, nb, 8, 32)
    mn = x.amin(dim=-1).clamp(max=0.0)
    mx = x.amax(dim=-1)
    scales, mins = (mx - mn) / 15.0, -mn                                   # [rows, nb, 8]
    d = (scales.amax(dim=-1, keepdim=True) / 63.0).to(torch.float16)
    dm = (mins.amax(dim=-1, keepdim=True) / 63.0).to(torch.float16)
    df, dmf = d.float(), dm.float()
    ls = torch.where(df > 0, _round_half_away(scales / df), torch.zeros_like(scales)).clamp_(0, 63)
    lm = torch.where(dmf > 0, _round_half_away(mins / dmf), torch.zeros_like(mins)).clamp_(0, 63)
    dl, ml = (df * ls).unsqueeze(-1), (dmf * lm).unsqueeze(-1)
    L = torch.where(dl > 0, _round_half_away((x + ml) / dl), torch.zeros_like(x)).clamp_(0, 15).to(torch.uint8)
    ls, lm = ls.to(torch.uint8), lm.to(torch.uint8)
    out = torch.zeros(rows, nb, 144, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = d.view(torch.uint8).reshape(rows, nb, 2)
    out[..., 2:4] = dm.view(torch.uint8).reshape(rows, nb, 2)
    sc = out[..., 4:16]
    sc[..., 0:4] = ls[..., 0:4] | ((ls[..., 4:8] >> 4) << 6)
    sc[..., 4:8] = lm[..., 0:4] | ((lm[..., 4:8] >> 4) << 6)
    sc[..., 8:12] = (ls[..., 4:8] & 0xF) | ((lm[..., 4:8] & 0xF) << 4)
    pairs = L.reshape(rows, nb, 4, 2, 32)                                  # 64-value groups: low nibbles then high
    out[..., 16:144] = (pairs[..., 0, :] | (pairs[..., 1, :] << 4)).reshape(rows, nb, 128)
    return out.reshape(rows, -1)


ENCODERS = {"Q4_K": quantize_q4_k, "Q8_0": quantize_q8_0}
