"""Beam search over the driver: beams are sequences that share the K/V blocks of their common prefix.

``Driver`` rows are forked copy-on-write: full blocks are shared by reference count, the partial last block is
copied on the device, the rest of the reservation is fresh.  Each step runs every live beam as one batch, reads the
whole-vocabulary logits of the sampling rows, and keeps the ``width`` best (parent, token) pairs by summed
log-probability (crates/poot-llm/src/driver/step.rs:1322-1359 `beam`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from .driver import Driver, DriverError, NoFreeRow, Sequence_
from .kvcache import BLOCK, blocks_for
from .sampler import SamplingParams


def fork(d: Driver, seq_id: int) -> int:
    """A new sequence with the same tokens and K/V as ``seq_id`` (which must have no pending tokens)."""
    s = d.seqs[seq_id]
    if s.pending != 0:
        raise DriverError("fork a sequence between a step and its commit (no pending tokens)")
    if not d._free_rows:
        raise NoFreeRow("no free serving row for the fork")
    full = s.computed // BLOCK
    fresh = d.pool.alloc(len(s.blocks) - full)
    for b in s.blocks[:full]:
        d.pool.retain(b)
    if s.computed % BLOCK:
        d.engine.copy_block(s.blocks[full], fresh[0])
    row = d._free_rows.pop()
    sid = next(d._ids)
    import copy
    n = Sequence_(sid, row, list(s.tokens), s.prompt_len, copy.copy(s.params), s.blocks[:full] + fresh, s.identity,
                  computed=s.computed, cached_tokens=s.cached_tokens, generated=s.generated, counts=dict(s.counts),
                  seed=s.seed)
    # what the sequence runs under travels with the fork: its resident adapter, the rows that stand in for prompt
    # embeddings (a fork taken mid-prompt still has them ahead) and the rotary offset of a sectioned rope
    n.adapter_slot, n.embed_pos, n.embed_rows = s.adapter_slot, s.embed_pos, s.embed_rows
    n.rope_prefix, n.rope_delta = s.rope_prefix, s.rope_delta
    d.seqs[sid] = n
    d.engine.write_block_table(row, n.blocks)
    return sid


@dataclass
class Beam:
    seq_id: int
    score: float
    tokens: List[int]


def _log_softmax(x: np.ndarray) -> np.ndarray:
    m = x.max(axis=-1, keepdims=True)
    return x - m - np.log(np.exp(x - m).sum(axis=-1, keepdims=True))


def beam_search(d: Driver, prompt: Sequence[int], width: int = 4, max_tokens: int = 32, length_penalty: float = 1.0,
                eos: Optional[int] = None) -> List[Beam]:
    """Returns finished hypotheses, best first (score = sum of log-probabilities / len ** length_penalty)."""
    if width < 1 or width > d.max_rows:
        raise DriverError(f"beam width {width} needs that many serving rows (have {d.max_rows})")
    eos = d.eos_token if eos is None else eos
    sp = SamplingParams(max_tokens=max_tokens, ignore_eos=True)
    live = [Beam(d.open(prompt, sp), 0.0, [])]
    done: List[Beam] = []

    def norm(b: Beam) -> float:
        return b.score / max(len(b.tokens), 1) ** length_penalty

    try:
        for _ in range(max_tokens):
            ids = [b.seq_id for b in live]
            while True:                      # the first iterations prefill the prompt; then every beam samples
                res = d.step(ids)
                if res and all(r.token is not None for r in res):
                    break
            rows = [r.seq_id for r in res if r.token is not None]
            lp = _log_softmax(d.engine.last_logits(len(rows)).astype(np.float64))
            cand = []
            for bi, sid in enumerate(rows):
                beam = next(b for b in live if b.seq_id == sid)
                top = np.argpartition(-lp[bi], min(width, lp.shape[1] - 1))[:width]
                for t in top:
                    cand.append((beam.score + float(lp[bi, t]), beam, int(t)))
            cand.sort(key=lambda c: (-c[0], c[1].seq_id, c[2]))
            keep = cand[:width]
            children = {}
            for score, parent, tok in keep:
                children.setdefault(parent.seq_id, []).append((score, tok))
            nxt: List[Beam] = []
            for b in live:
                kids = children.get(b.seq_id, [])
                if not kids:
                    d.release(b.seq_id, "preempted")
                    continue
                forks = [fork(d, b.seq_id) for _ in kids[1:]]
                for sid, (score, tok) in zip([b.seq_id] + forks, kids):
                    d.commit(sid, [tok])
                    nb = Beam(sid, score, b.tokens + [tok])
                    if tok == eos or d.finished(sid, tok):
                        d.release(sid, "preempted")
                        done.append(nb)
                    else:
                        nxt.append(nb)
            live = nxt
            if not live or (len(done) >= width and max(map(norm, done)) >= max(map(norm, live))):
                break
    finally:
        for b in live:
            if b.seq_id in d.seqs:
                d.release(b.seq_id, "preempted")
    done.extend(live)
    return sorted(done, key=lambda b: -norm(b))
