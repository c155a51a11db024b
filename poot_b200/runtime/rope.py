"""RoPE cos/sin tables for every frequency-scaling flavour the reference supports.

A table is ``[positions, rot/2]`` fp32 (the reference duplicates the halves, crates/poot-graph-ir/src/
rope_table.rs:1-10; the kernels index one half).  Flavours follow HF ``modeling_rope_utils`` as the reference
does (rope_table.rs:64-150): plain, linear, dynamic NTK, YaRN, llama3 NTK-by-parts, LongRoPE, proportional.
Angles are computed in float64 and rounded once, so CPU oracle and device share the same table bits.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.config import DecoderConfig, RopeScaling


def inv_frequencies(dim: int, theta: float, scaling: Optional[RopeScaling], positions: int,
                    freq_factors: Optional[Sequence[float]] = None) -> Tuple[np.ndarray, float]:
    """Inverse frequencies ``[dim/2]`` (float64) and the attention factor that scales the table."""
    half = dim // 2
    j = np.arange(half, dtype=np.float64)
    sc = scaling or RopeScaling()
    kind = sc.kind
    base = float(theta)
    att = 1.0
    if kind == "dynamic" and positions > sc.original_max_position:
        base = base * ((sc.factor * positions / sc.original_max_position) - (sc.factor - 1.0)) ** (dim / (dim - 2.0))
    inv = base ** (-2.0 * j / dim)
    if kind == "proportional":
        # the table spans the whole head; only the first ``proportion`` of the (i, i + dim/2) pairs rotate
        inv = np.where(j < int(sc.proportion * dim // 2), inv, 0.0)
    if kind == "linear" and sc.factor > 0:
        inv = inv / sc.factor
    elif kind == "llama3":
        low_wl = sc.original_max_position / sc.low_freq_factor
        high_wl = sc.original_max_position / sc.high_freq_factor
        wl = 2.0 * math.pi / inv
        smooth = (sc.original_max_position / wl - sc.low_freq_factor) / (sc.high_freq_factor - sc.low_freq_factor)
        blended = (1.0 - smooth) * inv / sc.factor + smooth * inv
        inv = np.where(wl > low_wl, inv / sc.factor, np.where(wl < high_wl, inv, blended))
    elif kind == "yarn":
        def corr_dim(rot):
            return dim * math.log(sc.original_max_position / (rot * 2.0 * math.pi)) / (2.0 * math.log(base))
        low = max(math.floor(corr_dim(sc.beta_fast)), 0)
        high = min(math.ceil(corr_dim(sc.beta_slow)), dim - 1)
        if low == high:
            high += 0.001
        ramp = np.clip((j - low) / (high - low), 0.0, 1.0)
        extrap_mask = 1.0 - ramp
        inv = (inv / sc.factor) * (1.0 - extrap_mask) + inv * extrap_mask
        att = sc.attention_factor if sc.attention_factor is not None else (
            1.0 if sc.factor <= 1 else 0.1 * math.log(sc.factor) + 1.0)
    elif kind == "longrope":
        factors = sc.long_factor if (positions > sc.original_max_position and sc.long_factor) else sc.short_factor
        if factors:
            inv = inv / np.asarray(factors, dtype=np.float64)
        # HF: scale = sqrt(1 + ln(max/original)/ln(original)) when max > original
        if positions > sc.original_max_position:
            att = math.sqrt(1.0 + math.log(positions / sc.original_max_position) / math.log(sc.original_max_position))
        if sc.attention_factor is not None:
            att = sc.attention_factor
    if freq_factors is not None and kind not in ("yarn",) and not (kind == "longrope" and (sc.short_factor or sc.long_factor)):
        inv = inv / np.asarray(freq_factors, dtype=np.float64)
    return inv, float(att)


def rope_tables(cfg: DecoderConfig, positions: int, freq_factors: Optional[Sequence[float]] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(cos, sin)`` fp32 CPU tensors of shape ``[positions, rot/2]``."""
    inv, att = inv_frequencies(cfg.rot, cfg.rope_theta, cfg.rope_scaling, positions, freq_factors)
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    cos = (np.cos(ang) * att).astype(np.float32)
    sin = (np.sin(ang) * att).astype(np.float32)
    return torch.from_numpy(cos), torch.from_numpy(sin)
