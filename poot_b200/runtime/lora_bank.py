"""Resident LoRA adapters selected per row of a step (the reference's per-request indexed contraction,
crates/poot-graph-plan/src/passes/lora.rs:1-7: ``y + scale[idx] * IndexedMatMul(IndexedMatMul(x, A, idx), B, idx)``).

Adapters live in slots.  For every layer and every projection site of the engine's fused layouts the bank keeps two
stacks, ``A[slots, R, in]`` and ``B[slots, out, R]`` (bf16, zero where an adapter does not target a projection, the
adapter's scale folded into ``B``):

* ``qkv``  - the fused q|k|v projection: ``A = [A_q; A_k; A_v]`` (rank 3r), ``B`` block-diagonal over the q, k and v rows;
* ``gu``   - the interleaved gate/up projection: ``A = [A_gate; A_up]`` (rank 2r), ``B`` rows interleaved like the weight;
* ``o``, ``down`` - as stored.

A step carries ``row_slot[T]`` (``-1`` = no adapter).  Each site costs two launches of the grouped skinny GEMM with one
group per row (the group's "expert" is the row's slot; a negative slot yields zeros) and one add: rows of different
adapters, and rows without one, share a step.  Ranks are padded to a multiple of 64 so the second contraction's K
extent is a whole tile.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..models.config import DecoderConfig
from ..ops import cuda_ops as K
from ..ops import moe_ops as M

SITES = ("qkv", "o", "gu", "down")


class LoraBankError(ValueError):
    pass


class LoraBank:
    def __init__(self, cfg: DecoderConfig, n_layers: int, slots: int, max_rank: int, max_tokens: int, device):
        if cfg.is_moe:
            raise LoraBankError("adapters over routed experts are not built")
        self.cfg, self.slots, self.max_rank, self.device = cfg, slots, max_rank, torch.device(device)
        H, F = cfg.hidden, cfg.ffn
        self.dims = {"qkv": (H, cfg.q_size + 2 * cfg.kv_size, 3), "o": (cfg.q_size, H, 1), "gu": (H, 2 * F, 2), "down": (F, H, 1)}
        self.rank = {s: -(-(m * max_rank) // 64) * 64 for s, (_, _, m) in self.dims.items()}
        bf = torch.bfloat16
        self.A: List[Dict[str, torch.Tensor]] = []
        self.B: List[Dict[str, torch.Tensor]] = []
        for _ in range(n_layers):
            self.A.append({s: torch.zeros(slots, self.rank[s], i, dtype=bf, device=self.device) for s, (i, o, m) in self.dims.items()})
            self.B.append({s: torch.zeros(slots, o, self.rank[s], dtype=bf, device=self.device) for s, (i, o, m) in self.dims.items()})
        self.names: List[Optional[str]] = [None] * slots
        self.row_slot = torch.full((max_tokens,), -1, dtype=torch.int32, device=self.device)
        self.xa = torch.zeros(max_tokens, max(self.rank.values()), dtype=bf, device=self.device)
        self.delta = torch.zeros(max_tokens, max(o for _, o, _ in self.dims.values()), dtype=bf, device=self.device)

    # ---- residency ---------------------------------------------------------------------------------------------
    def slot_of(self, name: str) -> int:
        if name not in self.names:
            raise LoraBankError(f"adapter {name!r} is not resident")
        return self.names.index(name)

    def load(self, adapter, layer0: int = 0) -> int:
        """Put a loaded adapter (``load.lora.LoraAdapter``) into a free slot; returns the slot."""
        if adapter.name in self.names:
            raise LoraBankError(f"adapter {adapter.name!r} is already resident")
        if adapter.rank > self.max_rank:
            raise LoraBankError(f"adapter rank {adapter.rank} exceeds the bank's {self.max_rank}")
        if None not in self.names:
            raise LoraBankError(f"all {self.slots} adapter slots are in use")
        slot = self.names.index(None)
        c, r = self.cfg, adapter.rank
        q, kv, F = c.q_size, c.kv_size, c.ffn
        known = set()
        for l in range(len(self.A)):
            p = f"layers.{layer0 + l}."

            def ab(role):
                known.add(p + role)
                return adapter.deltas.get(p + role)

            def put(site, a_rows, b_rows, b_cols, pair, interleave=None):
                if pair is None:
                    return
                a, b = pair
                self.A[l][site][slot, a_rows:a_rows + r] = torch.from_numpy(np.array(a)).to(torch.bfloat16)
                bs = torch.from_numpy(np.asarray(b * adapter.scale, dtype=np.float32)).to(torch.bfloat16)
                if interleave is None:
                    self.B[l][site][slot, b_rows:b_rows + bs.shape[0], b_cols:b_cols + r] = bs
                else:                                   # gate rows at even positions, up rows at odd ones
                    self.B[l][site][slot, interleave::2, b_cols:b_cols + r] = bs
            for s in SITES:
                self.A[l][s][slot].zero_()
                self.B[l][s][slot].zero_()
            put("qkv", 0, 0, 0, ab("attn_q"))
            put("qkv", r, q, r, ab("attn_k"))
            put("qkv", 2 * r, q + kv, 2 * r, ab("attn_v"))
            put("o", 0, 0, 0, ab("attn_o"))
            put("gu", 0, 0, 0, ab("ffn_gate"), interleave=0)
            put("gu", r, 0, r, ab("ffn_up"), interleave=1)
            put("down", 0, 0, 0, ab("ffn_down"))
        first, last = layer0, layer0 + len(self.A)
        stray = [k for k in adapter.deltas if k not in known and first <= int(k.split(".")[1]) < last]
        if stray:
            raise LoraBankError(f"adapter {adapter.name!r} targets {stray[0]}, which has no adapter site")
        self.names[slot] = adapter.name
        return slot

    def unload(self, name: str) -> None:
        self.names[self.slot_of(name)] = None

    # ---- per step ----------------------------------------------------------------------------------------------
    def bind_rows(self, rows: Optional[np.ndarray], T: int) -> bool:
        """Copy the step's row -> slot table; returns whether any row uses an adapter."""
        if rows is None:
            return False
        self.row_slot[:T].copy_(torch.from_numpy(np.ascontiguousarray(rows[:T], dtype=np.int32)))
        return bool((rows[:T] >= 0).any())

    def apply(self, eng, site: str, layer: int, x: torch.Tensor, out: torch.Tensor, T: int) -> None:
        """``out[:T] += B[slot] (A[slot] x)`` row by row (rows whose slot is negative get nothing)."""
        R = self.rank[site]
        N = self.dims[site][1]
        xa = self.xa[:T, :R]
        delta = self.delta[:T, :N]
        idx = self.row_slot[:T]
        eng._count(3)
        M.gemm_grouped(K.EPI_STORE, x, self.A[layer][site], self.xa, 1, T, group_expert=idx, x_row_mul=1,
                       out_group_stride=self.xa.stride(0), ldo=self.xa.stride(0))
        M.gemm_grouped(K.EPI_STORE, xa, self.B[layer][site], self.delta, 1, T, group_expert=idx, x_row_mul=1,
                       out_group_stride=self.delta.stride(0), ldo=self.delta.stride(0), K_dim=R)
        if delta.stride(0) == N and out.is_contiguous():
            K.add(out, delta, out=out)
        else:
            out.add_(delta)
