"""CPU oracle of the sampling rules (the semantics every device sampler must reproduce).

Definitions follow crates/poot-eval/src/ops/sampling.rs:40-183 and crates/poot-graph-ir/src/op.rs:118-189:
``hash32 = fmix32(seed ^ idx*0x9E3779B9)``, ``u = (2*(hash>>9)+1)*2^-24``, Gumbel noise ``-ln(-ln u)``,
perturbed score ``logit*inv_temp + noise_scale*noise`` with two roundings in f32, first index wins ties,
top-k by a 30-step value bisection from ``min_logit``, min-p floor ``max+floor_offset``, top-p by a 30-step
bisection over exact integer masses ``round(exp((l-max)*inv_temp)*2^24)``; the output is
``(token, non_finite_index)`` with the token forced to 0 when any logit is non-finite.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np

F32 = np.float32
MASKED_LOGIT = float(np.finfo(np.float32).min)
TOP_P_MASS_UNITS = F32(16777216.0)
GREEDY, GUMBEL, GUMBEL_TOPK, GUMBEL_TOPK_TOPP = 0, 1, 2, 3


def rule_for_truncation(top_k: int, top_p: float) -> int:
    """The rule a temperature draw's knobs select (``top_k == 0`` / ``top_p >= 1`` mean disabled)."""
    if top_p < 1.0:
        return GUMBEL_TOPK_TOPP
    if top_k > 0:
        return GUMBEL_TOPK
    return GUMBEL


def hash32(seed: int, idx: int) -> int:
    x = (seed ^ ((idx * 0x9E3779B9) & 0xFFFFFFFF)) & 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x85EBCA6B) & 0xFFFFFFFF
    x ^= x >> 13
    x = (x * 0xC2B2AE35) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def random_uniform_at(seed: int, idx: int) -> float:
    mant = hash32(seed & 0xFFFFFFFF, idx) >> 9
    return float((F32(2.0) * F32(mant) + F32(1.0)) * F32(5.9604645e-8))


def random_uniform_row(seed: int, cols: int) -> np.ndarray:
    idx = np.arange(cols, dtype=np.uint64)
    x = (np.uint64(seed & 0xFFFFFFFF) ^ ((idx * np.uint64(0x9E3779B9)) & np.uint64(0xFFFFFFFF))) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x85EBCA6B)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(13)
    x = (x * np.uint64(0xC2B2AE35)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    mant = (x >> np.uint64(9)).astype(np.float32)
    return (F32(2.0) * mant + F32(1.0)) * F32(5.9604645e-8)


def gumbel_noise(u: np.ndarray) -> np.ndarray:
    u = u.astype(np.float32)
    return -np.log(-np.log(u)).astype(np.float32)


def top_p_token_mass(logit: np.ndarray, max_logit, inv_temp) -> np.ndarray:
    e = np.exp(((logit.astype(np.float32) - F32(max_logit)) * F32(inv_temp)).astype(np.float32)).astype(np.float32)
    m = (e * TOP_P_MASS_UNITS).astype(np.float32)
    # round half away from zero, as Rust's f32::round
    return np.floor(m.astype(np.float64) + 0.5).astype(np.uint64)


def sample_one_row(logits: np.ndarray, noise: Optional[np.ndarray], params, top_k: Optional[int],
                   top_p: Optional[float]):
    logits = logits.astype(np.float32)
    finite = np.isfinite(logits)
    nf = np.nonzero(~finite)[0]
    flag = int(nf[0]) if nf.size else -1
    fin_vals = logits[finite]
    max_logit = F32(fin_vals.max()) if fin_vals.size else F32(np.finfo(np.float32).min)
    cand = fin_vals[fin_vals != F32(MASKED_LOGIT)]
    min_logit = F32(cand.min()) if cand.size else F32(np.finfo(np.float32).max)
    if params is None:
        if not fin_vals.size or flag >= 0:
            return 0, flag
        masked = np.where(finite, logits, -np.inf)
        return int(np.argmax(masked)), flag
    inv_temp, floor_offset, noise_scale = (F32(params[0]), F32(params[1]), F32(params[2]))
    with np.errstate(invalid="ignore", over="ignore"):
        lo = min_logit
        if top_k is not None and float(top_k) > 0.0:
            hi = max_logit
            for _ in range(30):
                mid = F32((lo + hi) * F32(0.5))
                count = int(np.count_nonzero(logits >= mid))
                if float(count) >= float(top_k):
                    lo = mid
                else:
                    hi = mid
        t_k = lo
        min_p_floor = F32(max_logit + floor_offset)
        floor = min_p_floor if min_p_floor > t_k else t_k
        if top_p is not None:
            floor1 = floor
            tp = F32(top_p)
            if tp <= 0:
                floor = max_logit
            elif tp < 1:
                def mass_at(th):
                    sel = logits >= th
                    return int(top_p_token_mass(logits[sel], max_logit, inv_temp).sum())
                total = mass_at(floor1)
                thresh = int(math.floor(float(F32(tp * F32(total))) + 0.5))
                tlo, thi = floor1, max_logit
                for _ in range(30):
                    mid = F32((tlo + thi) * F32(0.5))
                    if mass_at(mid) >= thresh:
                        tlo = mid
                    else:
                        thi = mid
                floor = floor1 if floor1 > tlo else tlo
        keep = logits >= floor
        if not keep.any():
            return 0, flag
        scaled = (logits * inv_temp).astype(np.float32)
        pert = (scaled + (noise_scale * noise.astype(np.float32)).astype(np.float32)).astype(np.float32)
        pert = np.where(keep, pert, -np.inf)
        best = int(np.argmax(pert))  # first maximum
    token = 0 if flag >= 0 else best
    return token, flag


def sample_rows(logits: np.ndarray, params: Optional[np.ndarray], top_k: Optional[np.ndarray],
                seeds: Optional[np.ndarray], rule: int) -> np.ndarray:
    """``[rows, 2]`` int32 ``(token, non_finite_index)``; noise is drawn from ``seeds`` per row."""
    rows, vocab = logits.shape
    out = np.zeros((rows, 2), dtype=np.int32)
    for r in range(rows):
        if rule == GREEDY:
            out[r] = sample_one_row(logits[r], None, None, None, None)
            continue
        noise = gumbel_noise(random_uniform_row(int(seeds[r]), vocab))
        k = int(top_k[r]) if rule >= GUMBEL_TOPK else None
        tp = float(params[r][3]) if rule >= GUMBEL_TOPK_TOPP else None
        out[r] = sample_one_row(logits[r], noise, params[r][:3], k, tp)
    return out
