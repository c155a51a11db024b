"""Capacity fit: the largest (rows, max_seq) whose planned device bytes fit the memory that is free.

Candidates are the requested shape, then ``max_seq`` halved down to a floor of 128, then ``rows`` halved; each is
PLANNED (a size-only walk of every buffer the engine would allocate: the paged K/V pool, activations, logits,
sampler scratch, tensor-parallel exchange blocks, captured-graph reserve) and admitted against the free-memory
budget minus a 256 MiB reserve (crates/poot-llm/src/driver/capacity.rs:1-22,539,721).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from ..models.config import DecoderConfig
from .kvcache import BLOCK, blocks_for

RESERVE = 256 << 20
FLOOR_SEQ = 128


class DoesNotFit(ValueError):
    pass


@dataclass
class ServingShapes:
    rows: int
    max_seq: int
    prefill_chunk: int
    num_blocks: int
    planned_bytes: int
    kv_bytes: int

    @property
    def max_tokens(self) -> int:
        return max(self.prefill_chunk, self.rows) + self.rows


def kv_bytes_per_block(cfg: DecoderConfig, tp_world: int = 1, kv_itemsize: int = 2) -> int:
    hkv = max(cfg.n_kv_heads // tp_world, 1)
    index = cfg.n_layers * BLOCK * cfg.index_head_dim * 2 if cfg.index_topk else 0    # the sparse indexer's own key pool
    return cfg.n_layers * 2 * hkv * BLOCK * cfg.head_dim * kv_itemsize + index


def plan_bytes(cfg: DecoderConfig, rows: int, max_seq: int, prefill_chunk: int, num_blocks: int, tp_world: int = 1,
               kv_itemsize: int = 2, graphs: int = 32) -> int:
    """Bytes of every engine-owned buffer for this shape (mirrors ``DecoderEngine.__init__`` allocation by allocation)."""
    T = max(prefill_chunk, rows) + rows
    if tp_world > 1:
        T = max(T, 128)
    H, D = cfg.hidden, cfg.head_dim
    hq, hkv = cfg.n_heads // tp_world, max(cfg.n_kv_heads // tp_world, 1)
    ffn = cfg.moe_ffn if cfg.is_moe else cfg.ffn // tp_world
    small_T = min(T, 256)
    act = 2 * T * (2 * H + (hq + 2 * hkv) * D + 2 * hq * D + ffn)
    partials = 8 * small_T * H * 4
    logits = rows * cfg.vocab * 4 + 2 * rows * H * 2
    if tp_world > 1:
        vl = cfg.vocab // tp_world
        logits += max(rows, 128) * vl * 4 + rows * vl * 4 + tp_world * rows * vl * 4
        logits += (tp_world + 1) * 2 * 128 * H * 4            # exchange inbox + gather buffer of the fused path
    attn_scratch = small_T * hq * 16 * (D + 2) * 4
    tables = rows * blocks_for(max_seq) * 4 + 8 * T * 4
    rope = 2 * cfg.max_position * (cfg.rot // 2 if hasattr(cfg, "rot") else D // 2) * 4
    moe = 0
    if cfg.is_moe:
        moe = T * cfg.n_experts * 4 * 3 + cfg.top_k * T * (H + ffn) * 2 * 2
    graph_reserve = graphs * (1 << 20)
    return num_blocks * kv_bytes_per_block(cfg, tp_world, kv_itemsize) + act + partials + logits + attn_scratch + tables + \
        rope + moe + graph_reserve


def candidates(rows: int, max_seq: int) -> List[tuple]:
    out, s = [], max_seq
    while s >= FLOOR_SEQ:
        out.append((rows, s))
        s //= 2
    r = rows // 2
    while r >= 1:
        out.append((r, max(FLOOR_SEQ, out[-1][1])))
        r //= 2
    return out


def fit(cfg: DecoderConfig, free_bytes: int, rows: int, max_seq: int, prefill_chunk: int = 512, tp_world: int = 1,
        kv_itemsize: int = 2, kv_fraction: float = 1.0, reserve: int = RESERVE) -> ServingShapes:
    """First candidate that fits.  The K/V pool takes what is left (capped at ``rows`` full-length sequences) but
    never less than one full-length sequence plus one block."""
    budget = int(free_bytes * kv_fraction) - reserve
    per_block = kv_bytes_per_block(cfg, tp_world, kv_itemsize)
    max_seq = min(max_seq, cfg.max_position)
    for r, s in candidates(rows, max_seq):
        chunk = min(prefill_chunk, s)
        fixed = plan_bytes(cfg, r, s, chunk, 0, tp_world, kv_itemsize)
        floor_blocks = blocks_for(s) + 1
        if fixed + floor_blocks * per_block > budget:
            continue
        blocks = min((budget - fixed) // per_block, r * blocks_for(s) + 1)
        return ServingShapes(r, s, chunk, int(blocks), fixed + int(blocks) * per_block, int(blocks) * per_block)
    raise DoesNotFit(f"no serving shape down to rows=1, max_seq={FLOOR_SEQ} fits {free_bytes / 2**30:.1f} GiB free "
                     f"(reserve {reserve >> 20} MiB)")
