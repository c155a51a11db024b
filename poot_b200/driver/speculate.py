"""Speculative decoding for one greedy sequence: draft k tokens cheaply, verify them in ONE target step.

Draft policies (crates/poot-llm/src/driver/speculate.rs:1-20; website/docs/serve/speculative-decoding.md):
``LookupDraft`` proposes the continuation that followed the most recent earlier occurrence of the current n-gram
in the sequence itself (prompt lookup); ``ModelDraft`` runs a smaller model greedily.  Verification feeds
``[last token, d1 .. dk]`` as one piece with a logit row at each position; the accepted prefix is the run of drafts
equal to the target's own greedy picks, plus the target's pick after it, so the output is token-for-token what
plain greedy decoding produces.  Rejected drafts leave stale K/V in slots past the accepted length; those positions
are rewritten when their real tokens are fed and are never visible to attention before that.  Recurrent state is
different: a rejected draft has been folded into it and cannot be taken out again, so on a model with recurrent
mixers the round snapshots the sequence's state rows before the verify step and, after a partial accept, restores them
and replays the kept tokens (crates/poot-llm/src/driver/snapshot.rs:1-17).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from ..oracle import sampling as S
from .driver import Driver, DriverError, StepInputs, _bucket
from .kvcache import BLOCK


class LookupDraft:
    def __init__(self, ngram: int = 3, k: int = 4):
        if ngram < 1 or k < 1:
            raise ValueError("lookup drafting needs NGRAM >= 1 and K >= 1")
        self.ngram, self.k = ngram, k

    @staticmethod
    def parse(text: str) -> "LookupDraft":
        """``NGRAM:K`` as in ``--draft-lookup``."""
        a, sep, b = text.partition(":")
        if not sep or not a.isdigit() or not b.isdigit():
            raise ValueError(f"--draft-lookup {text!r}: expected NGRAM:K")
        return LookupDraft(int(a), int(b))

    def propose(self, tokens: Sequence[int]) -> List[int]:
        n = self.ngram
        if len(tokens) <= n:
            return []
        key = list(tokens[-n:])
        for start in range(len(tokens) - n - 1, -1, -1):     # most recent earlier occurrence
            if list(tokens[start:start + n]) == key:
                return list(tokens[start + n:start + n + self.k])
        return []


class ModelDraft:
    """Greedy continuation from a smaller model behind its own driver."""

    def __init__(self, draft_driver: Driver, k: int = 4):
        self.d, self.k = draft_driver, k

    def propose(self, tokens: Sequence[int]) -> List[int]:
        from .sampler import SamplingParams
        return self.d.generate(list(tokens), SamplingParams(max_tokens=self.k, ignore_eos=True))


class MtpDraft:
    """Drafts from the served model's own multi-token-prediction layer (crates/poot-llm/src/driver/speculate.rs:20-33).

    The layer is a one-block model of its own (``models.config.mtp_config``) behind ``runner``, a step engine that
    shares the target's block tables, so its K/V for a position lives at the slot the target uses for it.  At position
    ``p`` it reads the target's closing hidden state of ``p`` and the token that follows ``p``, and guesses the token
    after that.  After every target step the layer runs over the positions the step wrote (``catch_up``): its cache
    then holds every committed position, and the last position's pick is the first draft of the sequence's next round.
    The round's other ``k - 1`` drafts are one-token chain steps, each fed the draft before it and the layer's own
    closing state of the step before (the post-norm state: recycling the pre-norm one lowers acceptance).  Chain steps
    write cache entries past the committed prefix; they are masked by the context length until the next catch-up, which
    starts at the query position, overwrites them.  A sequence whose last result was not committed whole proposes
    nothing for a round.
    """

    def __init__(self, runner, k: int = 1):
        if k < 1:
            raise ValueError("multi-token-prediction drafting needs K >= 1")
        self.runner, self.k = runner, k
        self.next = {}              # seq id -> (position of the round's query token, query token, first draft, hidden row)
        self.stats = {"catch_up_steps": 0, "chain_steps": 0}

    def attach(self, d: Driver) -> "MtpDraft":
        """Share the target's block tables and run after each of its steps."""
        inner = getattr(d.engine, "inner", d.engine)
        if not getattr(inner, "carry", False):
            raise DriverError("the target engine exports no hidden-state carry for its multi-token-prediction layer")
        if hasattr(inner, "block_tables") and hasattr(self.runner, "block_tables"):
            self.runner.block_tables = inner.block_tables
        d.after_step = self.catch_up
        return self

    def _run(self, d: Driver, spans, carry_rows: np.ndarray, sample: Sequence[bool]):
        """One step of the layer over ``spans`` = (sequence, first position, count, tokens after).  Returns the picks of
        the sampling spans' last rows and the layer's closing hidden state of every row."""
        T = sum(n for _, _, n, _ in spans)
        B = max(1, sum(bool(x) for x in sample))
        Tp, Bp = _bucket(T, self.runner.max_tokens), _bucket(B, d.max_rows)
        tokens = np.zeros(Tp, np.int32); positions = np.zeros(Tp, np.int32); slots = np.full(Tp, -1, np.int32)
        row_seq = np.zeros(Tp, np.int32); row_ctx = np.zeros(Tp, np.int32)
        carry = np.zeros((Tp, carry_rows.shape[1]), np.float32)
        carry[:T] = carry_rows
        logit_idx = np.zeros(Bp, np.int64)
        off = b = 0
        for (s, p0, n, after), want in zip(spans, sample):
            for i in range(n):
                pos = p0 + i
                tokens[off + i], positions[off + i], slots[off + i] = after[i], pos, d._slot(s, pos)
                row_seq[off + i], row_ctx[off + i] = s.row, pos + 1
            if want:
                logit_idx[b] = off + n - 1
                b += 1
            off += n
        params = np.zeros((Bp, 4), np.float32); params[:, 0] = 1.0; params[:, 1] = -1e30; params[:, 3] = 1.0
        inp = StepInputs(tokens, positions, slots, row_seq, row_ctx, logit_idx, S.GREEDY, params, np.zeros(Bp, np.int32),
                         np.zeros(Bp, np.int32), None, False, T, max(b, 1), carry=carry)
        picked, _ = self.runner.run_step(inp)
        return picked, self.runner.last_hidden

    def catch_up(self, d: Driver, spans) -> None:
        """Run the layer over the positions a target step just wrote.  ``spans``: (sequence, first position, count,
        offset of the span's rows in the step, the token after each position - one short when the step did not sample)."""
        hidden = getattr(d.engine, "last_hidden", None)
        if hidden is None:
            return
        for sid in [i for i in self.next if i not in d.seqs]:
            del self.next[sid]
        rows, carry, sample = [], [], []
        for s, p0, n, off, after in spans:
            self.next.pop(s.id, None)
            m = min(n, len(after))           # a prefill piece that ends the known tokens without a sample: last row waits
            if m <= 0:
                continue
            rows.append((s, p0, m, after[:m]))
            carry.append(np.asarray(hidden[off:off + m], np.float32))
            sample.append(m == n and len(s.tokens) == p0 + n)      # the step sampled this row's next token
        if not rows:
            return
        picked, own = self._run(d, rows, np.concatenate(carry, 0), sample)
        self.stats["catch_up_steps"] += 1
        off = b = 0
        for (s, p0, m, after), want in zip(rows, sample):
            if want:
                self.next[s.id] = (p0 + m, int(after[-1]), int(picked[b, 0]), np.array(own[off + m - 1], np.float32))
                b += 1
            off += m

    def propose_for(self, d: Driver, s, limit: int) -> List[int]:
        st = self.next.pop(s.id, None)
        if st is None or limit < 1:
            return []
        pos, query, first, hid = st
        if s.computed != pos or len(s.tokens) != pos + 1 or s.tokens[-1] != query:
            return []                        # the result the draft followed was not committed whole
        drafts = [first]
        while len(drafts) < min(self.k, limit):
            picked, own = self._run(d, [(s, pos + len(drafts) - 1, 1, [drafts[-1]])], hid[None, :], [True])
            self.stats["chain_steps"] += 1
            drafts.append(int(picked[0, 0]))
            hid = np.array(own[0], np.float32)
        return drafts


def speculative_step(d: Driver, seq_id: int, draft) -> List[int]:
    """One verify step; returns the tokens to commit (>= 1).  The sequence must be greedy, unguided and past prefill."""
    s = d.seqs[seq_id]
    if not s.params.greedy or s.guided is not None or s.params.needs_adjust:
        raise DriverError("speculation verifies plain greedy sequences only")
    if s.pending != 1:
        raise DriverError("speculate after the prompt is prefilled (pending must be 1)")
    room = min(len(s.blocks) * BLOCK, d.max_seq_len) - len(s.tokens) - 1
    room = min(room, s.params.max_tokens - s.generated - 1)
    limit = max(0, min(room, d.max_rows - 1, d.engine.max_tokens - 1))
    drafts = draft.propose_for(d, s, limit) if hasattr(draft, "propose_for") else list(draft.propose(s.tokens))[:limit]
    if any(t < 0 or t >= d.vocab for t in drafts):
        drafts = []
    piece = [s.tokens[-1]] + drafts
    T, B = len(piece), len(piece)
    Tp, Bp = _bucket(T, d.engine.max_tokens), _bucket(B, d.max_rows)
    tokens = np.zeros(Tp, np.int32); positions = np.zeros(Tp, np.int32); slots = np.full(Tp, -1, np.int32)
    row_seq = np.zeros(Tp, np.int32); row_ctx = np.zeros(Tp, np.int32)
    base = s.computed
    for i, t in enumerate(piece):
        tokens[i], positions[i], slots[i] = t, base + i, d._slot(s, base + i)
        row_seq[i], row_ctx[i] = s.row, base + i + 1
    logit_idx = np.zeros(Bp, np.int64)
    logit_idx[:B] = np.arange(T)
    params = np.zeros((Bp, 4), np.float32); params[:, 0] = 1.0; params[:, 1] = -1e30; params[:, 3] = 1.0
    inp = StepInputs(tokens, positions, slots, row_seq, row_ctx, logit_idx, S.GREEDY, params, np.zeros(Bp, np.int32),
                     np.zeros(Bp, np.int32), None, False, T, B)
    recurrent = bool(drafts) and bool(getattr(d.engine, "has_recurrent_state", False))
    if recurrent:
        d.engine.snapshot_rows([s.row])
    picked, _ = d.engine.run_step(inp)
    d.stats["steps"] += 1
    accepted = 0
    while accepted < len(drafts) and int(picked[accepted, 0]) == drafts[accepted]:
        accepted += 1
    if recurrent and accepted < len(drafts):
        # the rejected drafts were folded into the recurrent state: take the rows back and replay what is kept
        d.engine.restore_rows([s.row])
        keep = 1 + accepted
        Tk = _bucket(keep, d.engine.max_tokens)
        rt = np.zeros(Tk, np.int32); rp = np.zeros(Tk, np.int32); rs = np.full(Tk, -1, np.int32)
        rq = np.zeros(Tk, np.int32); rc = np.zeros(Tk, np.int32)
        rt[:keep], rp[:keep], rs[:keep], rq[:keep], rc[:keep] = tokens[:keep], positions[:keep], slots[:keep], row_seq[:keep], row_ctx[:keep]
        li = np.zeros(_bucket(1, d.max_rows), np.int64)
        li[0] = keep - 1
        Bk = len(li)
        pk = np.zeros((Bk, 4), np.float32); pk[:, 0] = 1.0; pk[:, 1] = -1e30; pk[:, 3] = 1.0
        d.engine.run_step(StepInputs(rt, rp, rs, rq, rc, li, S.GREEDY, pk, np.zeros(Bk, np.int32), np.zeros(Bk, np.int32),
                                     None, False, keep, 1))
        d.stats["steps"] += 1
        d.stats["draft_replays"] = d.stats.get("draft_replays", 0) + 1
    out = drafts[:accepted] + [int(picked[accepted, 0])]
    if hasattr(draft, "catch_up"):
        # the verify step wrote positions base .. base + accepted for good; the layer catches up over them, fed the
        # accepted drafts and the target's own pick as the tokens that follow
        keep_tokens = s.tokens
        s.tokens = s.tokens + out[:-1]                  # what the sequence will hold once the caller commits the result
        try:
            draft.catch_up(d, [(s, base, 1 + accepted, 0, list(out))])
        finally:
            s.tokens = keep_tokens
    d.stats["decode_tokens"] += 1 + accepted
    d.stats["draft_proposed"] = d.stats.get("draft_proposed", 0) + len(drafts)
    d.stats["draft_accepted"] = d.stats.get("draft_accepted", 0) + accepted
    s.computed += 1 + accepted           # K/V of the fed token and of every accepted draft is final
    # commit all but the last through the driver (each commit appends the token; the next step feeds the last one)
    return out


def generate_speculative(d: Driver, prompt: Sequence[int], params, draft, on_token=None) -> List[int]:
    """Greedy generation with drafting; equals ``Driver.generate`` token for token."""
    sid = d.open(prompt, params)
    out: List[int] = []
    try:
        done = False
        while not done:
            s = d.seqs[sid]
            if s.pending > 1 or s.generated == 0:
                res = [r for r in d.step([sid]) if r.token is not None]
                toks = [res[0].token] if res else []
            else:
                toks = speculative_step(d, sid, draft)
            for k, t in enumerate(toks):
                d.commit(sid, [t])
                if k < len(toks) - 1:
                    pass                      # accepted drafts: their K/V is already in the cache
                out.append(t)
                if on_token is not None:
                    on_token(t)
                if d.finished(sid, t):
                    done = True
                    break
    finally:
        d.release(sid)
    return out
