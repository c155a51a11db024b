"""Minimal host-side step driver over :class:`DecoderEngine` for fixed batches (bench, smoke, tests).

It owns pinned host staging for the step inputs and a trivial block allocation (sequence ``i`` owns a
contiguous run of pool blocks).  The full open/step/commit/release driver with prefix caching lives in
``poot_b200.driver``; this class is the smallest public surface that exercises the same engine entry points:
``bind`` (H2D of the step inputs from pinned memory) -> ``run`` (graph replay) -> read ``picked`` (D2H).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .engine import KV_BLOCK, DecoderEngine, StepShape


class FixedBatchSession:
    def __init__(self, engine: DecoderEngine, batch: int, max_len: int):
        self.e = engine
        self.batch, self.max_len = batch, max_len
        self.blocks_per_seq = (max_len + KV_BLOCK - 1) // KV_BLOCK
        assert self.blocks_per_seq <= engine.max_blocks and batch <= engine.max_seqs
        assert batch * self.blocks_per_seq <= engine.kv.num_blocks
        bt = torch.arange(batch * self.blocks_per_seq, dtype=torch.int32).view(batch, self.blocks_per_seq)
        self.block_tables_host = bt.pin_memory() if torch.cuda.is_available() else bt
        engine.block_tables[:batch, :self.blocks_per_seq].copy_(self.block_tables_host)
        self.len_t = torch.zeros(batch, dtype=torch.int32)
        self._ar = torch.arange(batch, dtype=torch.int64)
        n = max(engine.max_tokens, batch)
        pin = torch.cuda.is_available()

        def buf(dtype):
            t = torch.zeros(n, dtype=dtype)
            return t.pin_memory() if pin else t

        self.h_tokens, self.h_pos, self.h_slots = buf(torch.int32), buf(torch.int32), buf(torch.int32)
        self.h_seq, self.h_ctx, self.h_lidx = buf(torch.int32), buf(torch.int32), buf(torch.int64)
        self.h_picked = torch.zeros(engine.max_seqs, 2, dtype=torch.int32)
        if pin:
            self.h_picked = self.h_picked.pin_memory()

    @property
    def lengths(self):
        return self.len_t.tolist()

    @lengths.setter
    def lengths(self, v):
        self.len_t = torch.as_tensor(list(v), dtype=torch.int32)

    def _slot(self, seq: int, pos: int) -> int:
        blk = int(self.block_tables_host[seq, pos // KV_BLOCK])
        return blk * KV_BLOCK + pos % KV_BLOCK

    def h2d_bytes(self, T: int, B: int) -> int:
        return T * 4 * 5 + B * 8

    def prefill(self, prompts: List[List[int]], sampler: int = 0) -> torch.Tensor:
        """Run whole prompts (all sequences in one step, chunked by the engine's token budget)."""
        assert len(prompts) == self.batch
        flat = [(s, p, tok) for s, pr in enumerate(prompts) for p, tok in enumerate(pr)]
        T = len(flat)
        assert T <= self.e.max_tokens, "prompt tokens exceed the engine's step token budget"
        for i, (s, p, tok) in enumerate(flat):
            self.h_tokens[i], self.h_pos[i], self.h_seq[i] = tok, p, s
            self.h_slots[i], self.h_ctx[i] = self._slot(s, p), p + 1
        off = 0
        for s, pr in enumerate(prompts):
            off += len(pr)
            self.h_lidx[s] = off - 1
        self.lengths = [len(pr) for pr in prompts]
        return self._step(StepShape(T, self.batch, sampler))

    def prefill_fast(self, tokens: torch.Tensor, sampler: int = 0) -> torch.Tensor:
        """Vectorised form of :meth:`prefill` for equal-length prompts given as an int32 ``[B, L]`` tensor."""
        B, L = tokens.shape
        assert B == self.batch and B * L <= self.e.max_tokens
        T = B * L
        pos = torch.arange(L, dtype=torch.int32).repeat(B)
        seq = torch.arange(B, dtype=torch.int32).repeat_interleave(L)
        self.h_tokens[:T] = tokens.reshape(-1)
        self.h_pos[:T], self.h_seq[:T] = pos, seq
        blk = self.block_tables_host[seq.long(), (pos // KV_BLOCK).long()]
        self.h_slots[:T] = blk * KV_BLOCK + pos % KV_BLOCK
        self.h_ctx[:T] = pos + 1
        self.h_lidx[:B] = torch.arange(B, dtype=torch.int64) * L + (L - 1)
        self.lengths = [L] * B
        return self._step(StepShape(T, B, sampler))

    def _bind_decode_inputs(self, tokens) -> None:
        B = self.batch
        pos = self.len_t
        self.h_tokens[:B] = torch.as_tensor(tokens, dtype=torch.int32)
        self.h_pos[:B] = pos
        blk = self.block_tables_host[self._ar, (pos // KV_BLOCK).long()]
        self.h_slots[:B] = blk * KV_BLOCK + pos % KV_BLOCK
        self.h_ctx[:B] = pos + 1
        self.h_seq[:B] = self._ar.to(torch.int32)
        self.h_lidx[:B] = self._ar

    def decode(self, tokens, sampler: int = 0) -> torch.Tensor:
        """One decode step: feed one token per sequence, return ``[B, 2]`` (token, non_finite_index) on host."""
        B = self.batch
        self._bind_decode_inputs(tokens)
        self.len_t = self.len_t + 1
        return self._step(StepShape(B, B, sampler))

    def _step(self, shape: StepShape) -> torch.Tensor:
        e, T, B = self.e, shape.tokens, shape.logit_rows
        e.bind(self.h_tokens[:T], self.h_pos[:T], self.h_slots[:T], self.h_seq[:T], self.h_ctx[:T], self.h_lidx[:B])
        e.run(shape)
        self.h_picked[:B].copy_(e.picked[:B], non_blocking=True)
        if e.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        return self.h_picked[:B]

    # ---- chained decode: N replays with no host round trip in between --------------------------------
    def decode_chain(self, first_tokens, steps: int, sampler: int = 0) -> None:
        """Device-chained greedy decode: the graph ends with the advance kernel, so replays need no inputs."""
        B = self.batch
        self._bind_decode_inputs(first_tokens)
        shape = StepShape(B, B, sampler, chain=True)
        self.e.prepare(shape)
        self.e.bind(self.h_tokens[:B], self.h_pos[:B], self.h_slots[:B], self.h_seq[:B], self.h_ctx[:B],
                    self.h_lidx[:B])
        for _ in range(steps):
            self.e.run(shape)
        self.len_t = self.len_t + steps
