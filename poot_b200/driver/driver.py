"""The sequence driver: open / step / commit / release over a step engine with a paged KV cache.

Mirrors the reference driver's contract (crates/poot-llm/src/driver/mod.rs:1-40, step.rs:393-1359):

* ``open``    reserves a row and the KV blocks for prompt + max_tokens (nothing is ever preempted), after matching
              the longest cached prefix of whole 16-token blocks;
* ``step``    plans every live row - a prefill piece (``prefill_chunk`` tokens, bin-packed into a per-step token
              budget of ``widest_piece + rows`` with one token reserved per decoding row, oldest first) or one
              decode token - pads the plan to a prepared step shape, runs ONE engine step and returns each row's
              sampled token (uncommitted);
* ``commit``  appends the kept tokens to the sequence;
* ``release`` frees the blocks and registers the prompt's full blocks in the prefix cache (not when preempted).

The engine behind it is any object with the small ``StepEngine`` surface, so the same driver runs on the device
engine, on the CPU oracle and on the recording fake used by the scheduling tests.
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

from ..oracle import sampling as S
from .kvcache import BLOCK, BASE_IDENTITY, BlockPool, OutOfBlocks, PrefixCache, blocks_for
from .sampler import SamplingParams, step_seed


class DriverError(RuntimeError):
    pass


class NoFreeRow(DriverError):
    """Every serving row is in use."""


class SamplerFault(DriverError):
    """The step produced a non-finite logit for this row (typed fault; the token is not committed)."""

    def __init__(self, seq_id: int, index: int):
        super().__init__(f"sequence {seq_id}: non-finite logit at index {index}")
        self.seq_id, self.index = seq_id, index


@dataclass
class StepInputs:
    """One engine step, already padded to a prepared shape (padding rows write nothing: slot -1, context 0)."""
    tokens: np.ndarray       # [T] int32
    positions: np.ndarray    # [T] int32
    slots: np.ndarray        # [T] int32, -1 = no KV write
    row_seq: np.ndarray      # [T] int32 row of the block table
    row_ctx: np.ndarray      # [T] int32 keys visible to the token (position + 1)
    logit_idx: np.ndarray    # [B] int64 index into the T tokens of each row that samples
    sampler: int             # 0 greedy, 1..3 Gumbel rule (widest needed by any row)
    params: np.ndarray       # [B, 4] f32
    top_k: np.ndarray        # [B] int32
    seeds: np.ndarray        # [B] int32
    adjust: Optional[dict] = None   # {"idx": [B, A] int32, "val": [B, A, 4] f32, "guided": {row: mask}}
    want_logprobs: bool = False
    live_tokens: int = 0
    live_rows: int = 0
    adapter_rows: Optional[np.ndarray] = None   # [T] int32 adapter slot of every token row (-1 = none); None = no row uses one
    embed_flags: Optional[np.ndarray] = None    # [T] int32, 1 = the token's embedding is replaced by its row of embed_rows
    embed_rows: Optional[np.ndarray] = None     # [T, hidden] f32 (rows without a flag are zero); None = no token is replaced
    rope_positions: Optional[np.ndarray] = None  # [3, T] int32 rotary position streams (time, row, column); None = the positions
    carry: Optional[np.ndarray] = None          # [T, hidden] f32: the hidden-state carry a multi-token-prediction layer reads


@dataclass
class RowResult:
    seq_id: int
    token: Optional[int]          # sampled token, or None while the prompt is still being prefilled
    consumed: int                 # tokens of the sequence processed by this step
    logprob: Optional[float] = None


@dataclass
class Sequence_:
    id: int
    row: int
    tokens: List[int]
    prompt_len: int
    params: SamplingParams
    blocks: List[int]
    identity: int = BASE_IDENTITY
    computed: int = 0             # tokens whose K/V is in the cache
    cached_tokens: int = 0        # served from the prefix cache at open
    generated: int = 0
    opened_at: float = field(default_factory=time.monotonic)
    counts: Dict[int, int] = field(default_factory=dict)   # token histogram for the penalties
    guided: Optional[object] = None                        # constraint object with .mask(vocab) / .advance(token)
    seed: int = 0
    adapter_slot: int = -1                                 # resident LoRA adapter of the sequence (-1 = base model)
    embed_pos: Optional[np.ndarray] = None                 # sorted prompt positions whose embeddings are replaced ...
    embed_rows: Optional[np.ndarray] = None                # ... by these rows [len(embed_pos), hidden] (image rows of a VLM)
    rope_prefix: Optional[np.ndarray] = None               # [3, prompt_len] rotary position streams of the prompt (sectioned rope)
    rope_delta: int = 0                                    # rotary position minus sequence index for every later token

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.computed


def chunk_plan(n: int, chunk: int, granule: int = 16) -> List[int]:
    """Pieces of a prompt of ``n`` tokens: full chunks, then descending powers of two of the granule, then the rest
    (crates/poot-llm/src/driver/chunks.rs:1-9) - a small set of distinct step shapes."""
    out = []
    while n >= chunk:
        out.append(chunk)
        n -= chunk
    p = chunk // 2
    while p >= granule and n > 0:
        if n >= p:
            out.append(p)
            n -= p
        p //= 2
    if n > 0:
        out.append(n)
    return out


def _bucket(n: int, cap: int) -> int:
    """Step shapes are padded to powers of two (and to the cap above the last one): few distinct captured graphs."""
    b = 1
    while b < n:
        b *= 2
    return b if b <= cap else max(cap, n)


class Driver:
    MAX_ADJ = 1024

    def __init__(self, engine, num_blocks: int, max_rows: int, max_seq_len: int, vocab: int, prefill_chunk: int = 512,
                 prefix_caching: bool = True, eos_token: Optional[int] = None, prefill_budget: Optional[int] = None):
        # every step is a guarded transaction: validation before launch, NeedsReset after a failure, Poisoned when the
        # clean-up fails too (runtime/lifecycle.py)
        from ..runtime.lifecycle import GuardedStepEngine, StepLimits
        if not isinstance(engine, GuardedStepEngine):
            engine = GuardedStepEngine(engine, StepLimits.of(engine, vocab), on_reset=self._drop_everything)
        self.engine = engine
        self.pool = BlockPool(num_blocks)
        self.prefix = PrefixCache(self.pool) if prefix_caching else None
        self.max_rows, self.max_seq_len, self.vocab = max_rows, max_seq_len, vocab
        if prefill_chunk < BLOCK:
            # a piece that does not finish its prompt is cut on a block boundary; a chunk below one block could never advance
            raise DriverError(f"prefill_chunk {prefill_chunk} is smaller than the K/V block of {BLOCK} tokens")
        self.prefill_chunk = prefill_chunk
        # prefill tokens a step may carry: one chunk (the reference's budget, widest piece + rows) unless raised, in
        # which case several sequences' pieces share a step and the projections run at a larger, more efficient M
        self.prefill_budget = max(prefill_budget or prefill_chunk, prefill_chunk)
        self.eos_token = eos_token
        self.max_blocks_per_seq = blocks_for(max_seq_len)
        self.seqs: Dict[int, Sequence_] = {}
        self.after_step = None      # hook run after every step with the spans it wrote (a multi-token-prediction draft catches up)
        self._free_rows = list(range(max_rows - 1, -1, -1))
        self._ids = itertools.count(1)
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "prefix_hit_tokens": 0,
                      "prefix_query_tokens": 0, "padded_tokens": 0}

    # ------------------------------------------------------------------------------------------------ admission
    def can_open(self, prompt_len: int, max_tokens: int) -> bool:
        need = blocks_for(min(prompt_len + max_tokens, self.max_seq_len))
        free = self.pool.available
        return bool(self._free_rows) and need <= free + (self.prefix.reclaimable() if self.prefix is not None else 0)

    def open(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, identity: int = BASE_IDENTITY,
             guided=None, adapter_slot: int = -1, embeds=None, rope_positions=None) -> int:
        """``adapter_slot``: slot of a resident LoRA adapter the sequence runs with (-1 = the base model).  K/V computed
        under one adapter is not valid under another, so the prefix-cache identity is taken per slot.
        ``embeds``: ``(positions, rows[len(positions), hidden])``: rows of another modality that replace the embeddings
        of those prompt tokens (crates/poot-llm/src/driver: ``generate_with_inputs``).  The tokens at those positions are
        placeholders that say nothing about the rows, so the prefix-cache identity also covers the rows' content.
        ``rope_positions[3, len(prompt)]``: the prompt's rotary position streams under a sectioned rope (an image's
        tokens carry (start, start + row, start + column)); later tokens continue one past the largest value.  A token's
        K/V slot and causal order stay its index in the sequence."""
        params = params or SamplingParams()
        embed_pos = embed_rows = None
        if embeds is not None:
            embed_pos = np.asarray(embeds[0], dtype=np.int64).reshape(-1)
            embed_rows = np.ascontiguousarray(embeds[1], dtype=np.float32).reshape(len(embed_pos), -1)
            if len(embed_pos) and (np.any(np.diff(embed_pos) <= 0) or embed_pos[0] < 0 or embed_pos[-1] >= len(prompt)):
                raise DriverError("embedding rows must name distinct prompt positions in ascending order")
        rope_prefix = None
        if rope_positions is not None:
            rope_prefix = np.ascontiguousarray(rope_positions, dtype=np.int32).reshape(3, -1)
            if rope_prefix.shape[1] != len(prompt) or rope_prefix.min() < 0:
                raise DriverError("rotary position streams must give three non-negative values per prompt token")
        if adapter_slot >= 0 and identity == BASE_IDENTITY:
            identity = (BASE_IDENTITY ^ (0x9E3779B97F4A7C15 * (adapter_slot + 1))) & 0xFFFFFFFFFFFFFFFF
        if embed_pos is not None and len(embed_pos):
            import zlib
            digest = zlib.crc32(embed_rows.tobytes(), zlib.crc32(embed_pos.tobytes()))
            identity = (identity ^ (0xC2B2AE3D27D4EB4F * (digest + 1))) & 0xFFFFFFFFFFFFFFFF
        if rope_prefix is not None:
            import zlib
            identity = (identity ^ (0x165667B19E3779F9 * (zlib.crc32(rope_prefix.tobytes()) + 1))) & 0xFFFFFFFFFFFFFFFF
        params.validate()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise DriverError("empty prompt")
        if any(t < 0 or t >= self.vocab for t in prompt):
            raise DriverError("prompt token outside the vocabulary")
        total = len(prompt) + params.max_tokens
        if len(prompt) >= self.max_seq_len:
            raise DriverError(f"prompt of {len(prompt)} tokens does not fit max_seq_len {self.max_seq_len}")
        total = min(total, self.max_seq_len)
        if not self._free_rows:
            raise NoFreeRow("no free serving row")
        matched: List[int] = []
        if self.prefix is not None:
            matched = self.prefix.match(prompt, identity, self.max_blocks_per_seq)
            self.stats["prefix_query_tokens"] += len(prompt)
            self.stats["prefix_hit_tokens"] += len(matched) * BLOCK
        need = blocks_for(total) - len(matched)
        try:
            if need > self.pool.available and self.prefix is not None:
                self.prefix.evict_unused(need - self.pool.available)
            fresh = self.pool.alloc(need)
        except OutOfBlocks:
            for b in matched:
                self.pool.release(b)
            raise
        row = self._free_rows.pop()
        sid = next(self._ids)
        seq = Sequence_(sid, row, prompt, len(prompt), params, matched + fresh, identity,
                        computed=len(matched) * BLOCK, cached_tokens=len(matched) * BLOCK, guided=guided,
                        seed=params.seed if params.seed is not None else (sid * 2654435761) & 0x7FFFFFFF)
        seq.adapter_slot = int(adapter_slot)
        seq.embed_pos, seq.embed_rows = embed_pos, embed_rows
        if rope_prefix is not None:
            seq.rope_prefix, seq.rope_delta = rope_prefix, int(rope_prefix.max()) + 1 - len(prompt)
        for t in prompt:
            seq.counts[t] = seq.counts.get(t, 0) + 1
        self.seqs[sid] = seq
        self.engine.write_block_table(row, seq.blocks)
        return sid

    def resume(self, seq_id: int, more_tokens: Sequence[int], extra_max_tokens: int = 0) -> None:
        """Append the next turn's tokens to a live sequence; its K/V stays (conversation mode)."""
        seq = self.seqs[seq_id]
        seq.tokens.extend(int(t) for t in more_tokens)
        seq.params.max_tokens = seq.generated + extra_max_tokens if extra_max_tokens else seq.params.max_tokens
        need = blocks_for(min(len(seq.tokens) + max(extra_max_tokens, 1), self.max_seq_len)) - len(seq.blocks)
        if need > 0:
            seq.blocks.extend(self.pool.alloc(need))
            self.engine.write_block_table(seq.row, seq.blocks)

    # ------------------------------------------------------------------------------------------------ stepping
    def plan(self, seq_ids: Optional[Iterable[int]] = None):
        """Rows of the next step: ``[(seq, piece)]`` oldest first under the token budget."""
        live = [self.seqs[i] for i in (seq_ids if seq_ids is not None else sorted(self.seqs))]
        live = [s for s in live if s.pending > 0]
        decode = [s for s in live if s.pending == 1]
        prefill = [s for s in live if s.pending > 1]
        widest = min(max((s.pending for s in prefill), default=0), self.prefill_chunk)
        if self.prefill_budget > self.prefill_chunk:
            widest = max(widest, min(sum(min(s.pending, self.prefill_chunk) for s in prefill), self.prefill_budget))
        budget = min(widest + len(live), self.engine.max_tokens)
        rows = [(s, 1) for s in decode]
        used = len(decode)
        for s in prefill:                       # FIFO best-effort bin packing
            piece = min(s.pending, self.prefill_chunk, budget - used)
            if piece <= 0:
                continue
            if piece < s.pending:               # keep chunk boundaries on block multiples
                piece = (piece // BLOCK) * BLOCK
                if piece == 0:
                    continue
            rows.append((s, piece))
            used += piece
        rows.sort(key=lambda r: r[0].id)
        return rows

    def _slot(self, seq: Sequence_, pos: int) -> int:
        return seq.blocks[pos // BLOCK] * BLOCK + pos % BLOCK

    def build_inputs(self, rows) -> StepInputs:
        T = sum(p for _, p in rows)
        sampling_rows = [(s, p) for s, p in rows if p == s.pending]
        B = len(sampling_rows)
        Tp = _bucket(T, self.engine.max_tokens)
        Bp = _bucket(max(B, 1), self.max_rows)
        tokens = np.zeros(Tp, np.int32); positions = np.zeros(Tp, np.int32); slots = np.full(Tp, -1, np.int32)
        row_seq = np.zeros(Tp, np.int32); row_ctx = np.zeros(Tp, np.int32)
        logit_idx = np.zeros(Bp, np.int64)
        params = np.zeros((Bp, 4), np.float32); params[:, 0] = 1.0; params[:, 1] = -1e30; params[:, 3] = 1.0
        top_k = np.zeros(Bp, np.int32); seeds = np.zeros(Bp, np.int32)
        rule, off, b = S.GREEDY, 0, 0
        adjust_rows, guided_rows, want_lp = {}, {}, False
        adapter_rows = np.full(Tp, -1, np.int32) if any(s.adapter_slot >= 0 for s, _ in rows) else None
        embed_flags = embed_vals = None
        rope_pos = np.zeros((3, Tp), np.int32) if any(s.rope_prefix is not None for s, _ in rows) else None
        for s, piece in rows:
            p0 = s.computed
            if rope_pos is not None:
                idx = np.arange(p0, p0 + piece)
                n_pre = 0 if s.rope_prefix is None else max(0, min(piece, s.rope_prefix.shape[1] - p0))
                if n_pre:
                    rope_pos[:, off:off + n_pre] = s.rope_prefix[:, p0:p0 + n_pre]
                rope_pos[:, off + n_pre:off + piece] = idx[n_pre:] + s.rope_delta
            if adapter_rows is not None:
                adapter_rows[off:off + piece] = s.adapter_slot
            if s.embed_pos is not None and p0 < s.prompt_len:
                lo, hi = np.searchsorted(s.embed_pos, (p0, p0 + piece))
                if hi > lo:
                    if embed_flags is None:
                        embed_flags = np.zeros(Tp, np.int32)
                        embed_vals = np.zeros((Tp, s.embed_rows.shape[1]), np.float32)
                    at = off + (s.embed_pos[lo:hi] - p0)
                    embed_flags[at] = 1
                    embed_vals[at] = s.embed_rows[lo:hi]
            if piece == 1:       # decode row: scalar stores (a numpy slice per row would cost more than the row)
                tokens[off], positions[off], row_seq[off], row_ctx[off] = s.tokens[p0], p0, s.row, p0 + 1
                slots[off] = s.blocks[p0 // BLOCK] * BLOCK + p0 % BLOCK
            else:                # prefill piece: one vectorised fill
                pos = np.arange(p0, p0 + piece, dtype=np.int32)
                sl = slice(off, off + piece)
                tokens[sl] = s.tokens[p0:p0 + piece]
                positions[sl] = pos
                slots[sl] = np.asarray(s.blocks, dtype=np.int32)[pos // BLOCK] * BLOCK + pos % BLOCK
                row_seq[sl] = s.row
                row_ctx[sl] = pos + 1
            if piece == s.pending:
                logit_idx[b] = off + piece - 1
                sp = s.params
                rule = max(rule, sp.rule)
                params[b] = sp.device_params()
                top_k[b] = sp.top_k if not sp.greedy else 0
                seeds[b] = step_seed(s.seed, s.generated)
                if sp.needs_adjust:
                    adjust_rows[b] = s
                if s.guided is not None:
                    # an engine with a late-input point builds the mask while the device runs the model body
                    guided_rows[b] = ((lambda g=s.guided: g.mask(self.vocab)) if getattr(self.engine, "late_inputs", False)
                                      else s.guided.mask(self.vocab))
                want_lp = want_lp or sp.logprobs > 0
                b += 1
            off += piece
        adjust = None
        if adjust_rows or guided_rows:
            idx = np.full((Bp, self.MAX_ADJ), -1, np.int32)
            val = np.zeros((Bp, self.MAX_ADJ, 4), np.float32)
            for r, s in adjust_rows.items():
                sp = s.params
                ents: Dict[int, List[float]] = {}
                for t, bias in sp.logit_bias.items():
                    ents[int(t)] = [float(bias), 1.0, 1.0, 0.0]
                for t, c in list(s.counts.items())[-self.MAX_ADJ:]:
                    # order of the reference: +bias, repetition on the biased value, then the additive penalties
                    e = ents.setdefault(t, [0.0, 1.0, 1.0, 0.0])
                    e[1] *= 1.0 / sp.repeat_penalty
                    e[2] *= sp.repeat_penalty
                    e[3] -= sp.presence_penalty + sp.frequency_penalty * c
                for k, (t, e) in enumerate(list(ents.items())[:self.MAX_ADJ]):
                    idx[r, k] = t
                    val[r, k] = e
            adjust = {"idx": idx, "val": val, "guided": guided_rows}
        from ..ir.analysis import check_write_slots
        check_write_slots(slots[:T])            # two rows writing one K/V slot in a step would race on the device
        self.stats["padded_tokens"] += Tp - T
        return StepInputs(tokens, positions, slots, row_seq, row_ctx, logit_idx, rule, params, top_k, seeds, adjust,
                          want_lp, T, B, adapter_rows, embed_flags, embed_vals, rope_pos)

    def step(self, seq_ids: Optional[Iterable[int]] = None) -> List[RowResult]:
        rows = self.plan(seq_ids)
        if not rows:
            return []
        inp = self.build_inputs(rows)
        picked, logprobs = self.engine.run_step(inp)
        self.stats["steps"] += 1
        out, b = [], 0
        spans, off = [], 0
        for s, piece in rows:
            sampled = piece == s.pending
            spans.append([s, s.computed, piece, off, list(s.tokens[s.computed + 1:s.computed + piece + 1])])
            off += piece
            s.computed += piece
            if piece > 1 or s.generated == 0 and not sampled:
                self.stats["prefill_tokens"] += piece
            else:
                self.stats["decode_tokens"] += piece
            if sampled and s.generated == 0 and self.prefix is not None:
                # the prompt's K/V is complete: later arrivals may share its full blocks while this one still decodes
                n_full = min(s.prompt_len, s.computed) // BLOCK
                self.prefix.register(s.tokens[:n_full * BLOCK], s.blocks[:n_full], s.identity)
            if sampled:
                tok, bad = int(picked[b, 0]), int(picked[b, 1])
                lp = float(logprobs[b]) if logprobs is not None else None
                b += 1
                if bad >= 0:
                    raise SamplerFault(s.id, bad)
                spans[-1][4].append(tok)
                out.append(RowResult(s.id, tok, piece, lp))
            else:
                out.append(RowResult(s.id, None, piece))
        if self.after_step is not None:
            # (sequence, first position, positions written, offset of its rows in the step, the token after each position)
            self.after_step(self, [tuple(sp) for sp in spans])
        return out

    def reset(self) -> None:
        """Complete reset after a failed step (``NeedsReset``): the engine restores its state and every open sequence,
        its blocks and the prefix cache are dropped, because K/V written by the failed step cannot be trusted."""
        self.engine.reset()

    def _drop_everything(self) -> None:
        for sid in list(self.seqs):
            s = self.seqs.pop(sid)
            for b in s.blocks:
                self.pool.release(b)
            self._free_rows.append(s.row)
        if self.prefix is not None:
            self.prefix.evict_unused(0)

    def commit(self, seq_id: int, tokens: Sequence[int]) -> None:
        s = self.seqs[seq_id]
        for t in tokens:
            if len(s.tokens) >= self.max_seq_len or len(s.tokens) >= len(s.blocks) * BLOCK:
                raise DriverError(f"sequence {seq_id} is at its reserved capacity")
            s.tokens.append(int(t))
            s.counts[int(t)] = s.counts.get(int(t), 0) + 1
            s.generated += 1
            if s.guided is not None:
                s.guided.advance(int(t))

    def finished(self, seq_id: int, token: int) -> Optional[str]:
        """Why the sequence ends after ``token`` was committed ("stop", "length") or None."""
        s = self.seqs[seq_id]
        sp = s.params
        if not sp.ignore_eos and self.eos_token is not None and token == self.eos_token:
            return "stop"
        if token in sp.stop_token_ids:
            return "stop"
        if s.guided is not None and getattr(s.guided, "done", lambda: False)():
            return "stop"
        if s.generated >= sp.max_tokens or len(s.tokens) >= self.max_seq_len:
            return "length"
        return None

    def release(self, seq_id: int, reason: str = "finished") -> dict:
        s = self.seqs.pop(seq_id)
        registered = 0
        if reason == "finished" and self.prefix is not None:
            n_full = min(s.prompt_len, s.computed) // BLOCK
            registered = self.prefix.register(s.tokens[:n_full * BLOCK], s.blocks[:n_full], s.identity)
        for b in s.blocks:
            self.pool.release(b)
        self._free_rows.append(s.row)
        return {"registered_tokens": registered, "generated": s.generated, "cached_tokens": s.cached_tokens}

    # ------------------------------------------------------------------------------------------------ convenience
    def generate(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, on_token=None, embeds=None,
                 rope_positions=None) -> List[int]:
        sid = self.open(prompt, params, embeds=embeds, rope_positions=rope_positions)
        out: List[int] = []
        try:
            while True:
                res = [r for r in self.step([sid]) if r.seq_id == sid]
                if not res:
                    break
                r = res[0]
                if r.token is None:
                    continue
                self.commit(sid, [r.token])
                out.append(r.token)
                if on_token is not None:
                    on_token(r.token)
                if self.finished(sid, r.token):
                    break
        finally:
            self.release(sid)
        return out

    def kv_usage(self) -> dict:
        total = self.pool.num_blocks
        return {"blocks_total": total, "blocks_used": total - self.pool.available,
                "usage_ratio": (total - self.pool.available) / max(total, 1),
                "prefix_entries": len(self.prefix) if self.prefix is not None else 0}
