"""Step engines behind the driver: the device engine adapter and the recording fake.

``DeviceStepEngine`` binds a padded ``StepInputs`` into the device engine's static buffers (one pinned staging
copy per field), replays the prepared step graph and reads back ``(token, non_finite_index)`` per sampling row -
never the logits (crates/poot-llm/src/driver/step.rs:776, suffix.rs:255).  ``FakeStepEngine`` records every step
and answers deterministically, which is how the scheduling and admission logic is tested without a GPU (the
reference's recording ``ServeEngine``, crates/poot-serve/src/tests/recording_engine.rs).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np

from .driver import StepInputs


class FakeStepEngine:
    """Next token = (last fed token of the row + 1) mod vocab (moved to the next token a guided mask allows);
    records the steps it was asked to run."""

    def __init__(self, vocab: int = 1000, max_tokens: int = 256, fail_at_step: Optional[int] = None):
        self.vocab, self.max_tokens = vocab, max_tokens
        self.steps: List[StepInputs] = []
        self.block_tables = {}
        self.fail_at_step = fail_at_step

    def write_block_table(self, row: int, blocks) -> None:
        self.block_tables[row] = list(blocks)

    def run_step(self, inp: StepInputs) -> Tuple[np.ndarray, Optional[np.ndarray]]:
        if self.fail_at_step is not None and len(self.steps) == self.fail_at_step:
            raise RuntimeError("injected engine fault")
        self.steps.append(inp)
        self.last_run_ms, self.last_device_ms, self.last_launches = 0.0, None, 0
        self._last_first = []
        B = len(inp.logit_idx)
        picked = np.zeros((B, 2), np.int32)
        picked[:, 1] = -1
        for b in range(inp.live_rows):
            tok = (int(inp.tokens[inp.logit_idx[b]]) + 1) % self.vocab
            mask = (inp.adjust or {}).get("guided", {}).get(b) if inp.adjust else None
            if mask is not None:      # a guided row: the first allowed token at or after the candidate, cyclically
                ok = np.flatnonzero(np.asarray(mask) == 0.0)
                later = ok[ok >= tok]
                tok = int(later[0] if len(later) else ok[0])
            picked[b, 0] = tok
            self._last_first.append((int(inp.tokens[inp.logit_idx[b]]) + 1) % self.vocab)
        return picked, (np.zeros(B, np.float32) if inp.want_logprobs else None)


    def last_logits(self, rows: int) -> np.ndarray:
        """Synthetic logits of the last step: the favourite scores 0, every next id half a nat less."""
        out = np.zeros((rows, self.vocab), np.float32)
        ids = np.arange(self.vocab)
        for b in range(rows):
            out[b] = -0.5 * ((ids - self._last_first[b]) % self.vocab)
        return out

    def copy_block(self, src: int, dst: int) -> None:
        self.copies = getattr(self, "copies", []) + [(src, dst)]


class DeviceStepEngine:
    """Adapter from ``StepInputs`` to :class:`poot_b200.runtime.engine.DecoderEngine`."""

    def __init__(self, engine):
        import torch
        self.torch = torch
        self.e = engine
        self.max_tokens = engine.max_tokens
        n = engine.max_tokens
        pin = torch.cuda.is_available()

        def buf(shape, dtype):
            t = torch.zeros(shape, dtype=dtype)
            return t.pin_memory() if pin else t

        self.h_tokens, self.h_pos, self.h_slots = buf(n, torch.int32), buf(n, torch.int32), buf(n, torch.int32)
        self.h_seq, self.h_ctx = buf(n, torch.int32), buf(n, torch.int32)
        B = engine.max_seqs
        self.h_lidx = buf(B, torch.int64)
        self.h_params, self.h_topk, self.h_seeds = buf((B, 4), torch.float32), buf(B, torch.int32), buf(B, torch.int32)
        self.h_picked, self.h_logprobs = buf((B, 2), torch.int32), buf(B, torch.float32)
        self.h_bt = buf((engine.max_seqs, engine.max_blocks), torch.int32)
        self.device_timing = False           # bracket each step with CUDA events (opt-in: it adds a synchronisation)
        self.last_device_ms = None           # None = not measured
        self.last_run_ms = None
        self.last_launches = 0

    def write_block_table(self, row: int, blocks) -> None:
        n = len(blocks)
        self.h_bt[row, :n] = self.torch.as_tensor(blocks, dtype=self.torch.int32)
        self.e.block_tables[row, :n].copy_(self.h_bt[row, :n], non_blocking=True)

    def run_step(self, inp: StepInputs):
        from ..runtime.engine import StepShape
        torch, e = self.torch, self.e
        T, B = len(inp.tokens), len(inp.logit_idx)
        for dst, src in ((self.h_tokens, inp.tokens), (self.h_pos, inp.positions), (self.h_slots, inp.slots),
                         (self.h_seq, inp.row_seq), (self.h_ctx, inp.row_ctx)):
            dst[:T] = torch.from_numpy(src)
        self.h_lidx[:B] = torch.from_numpy(inp.logit_idx)
        e.bind(self.h_tokens[:T], self.h_pos[:T], self.h_slots[:T], self.h_seq[:T], self.h_ctx[:T], self.h_lidx[:B])
        if inp.sampler != 0:
            self.h_params[:B] = torch.from_numpy(inp.params)
            self.h_topk[:B] = torch.from_numpy(inp.top_k)
            self.h_seeds[:B] = torch.from_numpy(inp.seeds)
            e.samp_params[:B].copy_(self.h_params[:B], non_blocking=True)
            e.samp_topk[:B].copy_(self.h_topk[:B], non_blocking=True)
            e.samp_seeds[:B].copy_(self.h_seeds[:B], non_blocking=True)
        guided = False
        if inp.adjust is not None:
            if e.adj_idx is None:
                e._alloc_adjust()
            e.adj_idx[:B].copy_(torch.from_numpy(inp.adjust["idx"]), non_blocking=False)
            e.adj_val[:B].copy_(torch.from_numpy(inp.adjust["val"]), non_blocking=False)
            if inp.adjust["guided"]:
                guided = True
                e.guided_mask[:B].zero_()
                for r, m in inp.adjust["guided"].items():
                    e.guided_mask[r].copy_(torch.from_numpy(np.ascontiguousarray(m, dtype=np.float32)))
        shape = StepShape(T, B, inp.sampler, False, inp.adjust is not None, guided, inp.want_logprobs)
        import time as _time
        t0 = _time.perf_counter()
        ev = None
        if self.device_timing:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        e.run(shape)
        if ev is not None:
            ev[1].record()
        self.h_picked[:B].copy_(e.picked[:B], non_blocking=True)
        if inp.want_logprobs:
            self.h_logprobs[:B].copy_(e.logprobs[:B], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.last_run_ms = (_time.perf_counter() - t0) * 1e3
        self.last_device_ms = ev[0].elapsed_time(ev[1]) if ev is not None else None
        self.last_launches = e.launches_per_step.get(e._key(shape), 0)
        return self.h_picked[:B].numpy().copy(), (self.h_logprobs[:B].numpy().copy() if inp.want_logprobs else None)

    def last_logits(self, rows: int) -> np.ndarray:
        """Whole-vocabulary logits of the last step's sampling rows (single-rank engines only)."""
        if self.e.tp != 1:
            raise RuntimeError("ranks of a tensor-parallel engine hold vocabulary shards")
        return self.e.logits[:rows].float().cpu().numpy()

    def copy_block(self, src: int, dst: int) -> None:
        """Copy one K/V block in every layer (a forked sequence gets its own copy of the partial last block)."""
        self.e.kv.buf[:, :, dst].copy_(self.e.kv.buf[:, :, src])
