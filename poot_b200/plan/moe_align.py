"""Block-aligned grouping of (token, slot) rows by expert: the host-side statement of the reference's
``group_expert_rows`` pass (crates/poot-graph-plan/src/passes/group_expert_rows.rs:1-8), the analogue of vLLM's
``moe_align_block_size``.  Rows routed to one expert are made contiguous and every expert's run is padded to a
multiple of the row-tile, so a grouped GEMM walks whole tiles that each belong to exactly one expert."""
from __future__ import annotations

from typing import Tuple

import numpy as np


def group_expert_rows(ids: np.ndarray, n_experts: int, block: int) -> Tuple[np.ndarray, np.ndarray, int]:
    """``ids`` [rows, k] expert of every (token, slot).  Returns ``(sorted_rows, tile_expert, padded)``:
    ``sorted_rows`` [padded] = flat (token * k + slot) index of each grouped row or -1 for padding, stable within an
    expert; ``tile_expert`` [padded / block] = expert of each row tile."""
    flat = np.asarray(ids).reshape(-1)
    if flat.size and (flat.min() < 0 or flat.max() >= n_experts):
        raise ValueError("expert id out of range")
    order = np.argsort(flat, kind="stable")
    counts = np.bincount(flat, minlength=n_experts)
    padded_counts = (counts + block - 1) // block * block
    starts = np.concatenate([[0], np.cumsum(padded_counts)[:-1]])
    padded = int(padded_counts.sum())
    sorted_rows = np.full(padded, -1, dtype=np.int64)
    src = 0
    for e in range(n_experts):
        c = int(counts[e])
        sorted_rows[starts[e]:starts[e] + c] = order[src:src + c]
        src += c
    tile_expert = np.repeat(np.arange(n_experts), padded_counts // block).astype(np.int32)
    return sorted_rows, tile_expert, padded
