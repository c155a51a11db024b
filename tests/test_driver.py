"""Driver logic on the recording fake engine: admission, chunked prefill plan, token budget, prefix cache,
block accounting, typed failures - no GPU (the reference tests its serve loop the same way)."""
import numpy as np
import pytest

from poot_b200.driver.driver import Driver, DriverError, NoFreeRow, chunk_plan
from poot_b200.driver.engines import FakeStepEngine
from poot_b200.driver.kvcache import BLOCK, BlockPool, OutOfBlocks, PrefixCache, chain_hash, chain_root
from poot_b200.driver.sampler import SamplingParams


def make(num_blocks=64, rows=4, max_seq=256, chunk=64, vocab=1000, **kw):
    eng = FakeStepEngine(vocab=vocab, max_tokens=128)
    return Driver(eng, num_blocks, rows, max_seq, vocab, prefill_chunk=chunk, **kw), eng


def test_chunk_plan_uses_full_chunks_then_powers_of_two():
    assert chunk_plan(300, 128) == [128, 128, 32, 12]
    assert chunk_plan(16, 128) == [16]
    assert sum(chunk_plan(1000, 128)) == 1000


def test_generate_prefills_in_chunks_then_decodes():
    d, eng = make()
    out = d.generate(list(range(100)), SamplingParams(max_tokens=5))
    assert out == [100, 101, 102, 103, 104]
    live = [s.live_tokens for s in eng.steps]
    assert live[:2] == [64, 36] and live[2:] == [1, 1, 1, 1]
    assert all(len(s.tokens) & (len(s.tokens) - 1) == 0 for s in eng.steps)      # padded to power-of-two shapes
    assert eng.steps[0].slots[63] >= 0 and (eng.steps[1].slots[36:] == -1).all()  # padding never writes KV
    assert d.pool.available == 64 - len(d.prefix)                                  # only cached blocks stay held


def test_budget_reserves_one_token_per_decoding_row_and_packs_fifo():
    d, eng = make(rows=4, chunk=64)
    a = d.open(list(range(10)), SamplingParams(max_tokens=8))
    for _ in range(2):
        for r in d.step():
            if r.token is not None:
                d.commit(r.seq_id, [r.token])
    b = d.open(list(range(200, 330)), SamplingParams(max_tokens=8))
    rows = d.plan()
    pieces = {s.id: p for s, p in rows}
    assert pieces[a] == 1 and pieces[b] == 64
    res = d.step()
    assert {r.seq_id for r in res} == {a, b}
    assert [r for r in res if r.seq_id == b][0].token is None


def test_prefix_cache_reuses_whole_blocks_and_never_the_last_token():
    d, eng = make()
    prompt = list(range(40))
    d.generate(prompt, SamplingParams(max_tokens=2))
    assert len(d.prefix) == 2                                  # two full 16-token blocks registered
    n0 = len(eng.steps)
    d.generate(prompt, SamplingParams(max_tokens=2))
    assert eng.steps[n0].live_tokens == 40 - 32                # 32 tokens came from the cache
    assert d.stats["prefix_hit_tokens"] == 32
    # an exact multiple of the block still recomputes its last block (one token must run for logits)
    d2, eng2 = make()
    d2.generate(list(range(32)), SamplingParams(max_tokens=1))
    n0 = len(eng2.steps)
    d2.generate(list(range(32)), SamplingParams(max_tokens=1))
    assert eng2.steps[n0].live_tokens == 16


def test_prefix_identity_separates_adapters_and_collisions_are_misses():
    pool = BlockPool(8)
    pc = PrefixCache(pool)
    toks = list(range(48))
    blocks = pool.alloc(3)
    assert pc.register(toks, blocks, identity=0) == 48
    assert pc.match(toks + [1], identity=7) == []                # other weights identity: no sharing
    assert pc.match(toks + [1], identity=0) == blocks
    pc.force_collisions(True)
    other = [t + 500 for t in toks]
    assert pc.match(other + [1], identity=0) == []               # same hash, different tokens -> miss
    for b in blocks:
        pool.release(b); pool.release(b)                         # sequence's and the match's references
    assert pool.available == 5 and pc.evict_unused() == 3 and pool.available == 8
    assert chain_hash(chain_root(), toks[:16]) != chain_hash(chain_root(), other[:16])


def test_admission_failures_are_typed_and_leave_no_leaks():
    d, _ = make(num_blocks=4, rows=2, max_seq=128)
    with pytest.raises(OutOfBlocks):
        d.open(list(range(60)), SamplingParams(max_tokens=60))
    assert d.pool.available == 4 and len(d.seqs) == 0
    a = d.open([1, 2, 3], SamplingParams(max_tokens=4))
    b = d.open([4, 5, 6], SamplingParams(max_tokens=4))
    with pytest.raises(NoFreeRow):
        d.open([7], SamplingParams(max_tokens=1))
    with pytest.raises(DriverError):
        d.open([], SamplingParams())
    with pytest.raises(DriverError):
        d.open([5000], SamplingParams())
    d.release(a, "preempted"); d.release(b)
    assert d.pool.available == 4 and len(d.prefix) == 0          # prompts shorter than a block cache nothing


def test_engine_fault_propagates_and_sequence_can_be_released():
    eng = FakeStepEngine(fail_at_step=1)
    d = Driver(eng, 16, 2, 128, 1000, prefill_chunk=64)
    sid = d.open(list(range(20)), SamplingParams(max_tokens=4))
    (r,) = d.step()
    d.commit(sid, [r.token])
    with pytest.raises(RuntimeError, match="injected"):
        d.step()
    d.release(sid, "preempted")
    assert d.pool.available + len(d.prefix) == 16          # the prompt's full block stays cached, everything else is free


def test_sampling_params_encode_rules_and_adjustments():
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.05, repeat_penalty=1.1, logit_bias={5: 2.0})
    assert sp.rule == 3 and SamplingParams(temperature=0.7, top_p=1.0, top_k=0).rule == 1 and SamplingParams().rule == 0
    inv_t, floor, ns, tp = sp.device_params()
    assert abs(inv_t - 1.25) < 1e-6 and floor < 0 and ns == 1.0 and tp == 0.9
    d, eng = make()
    sid = d.open([5, 6, 5], sp)
    d.step()
    adj = eng.steps[-1].adjust
    row = {int(t): v for t, v in zip(adj["idx"][0], adj["val"][0]) if t >= 0}
    assert row[5][0] == 2.0 and abs(row[5][1] - 1 / 1.1) < 1e-6 and abs(row[6][2] - 1.1) < 1e-6
    with pytest.raises(ValueError):
        SamplingParams(top_p=1.5).validate()


def test_a_larger_prefill_budget_packs_several_pieces_into_one_step():
    from poot_b200.llm import LLM
    def steps(budget):
        llm = LLM.fake(vocab=5000, rows=8, max_seq=1024, num_blocks=8 * 64 + 8, prefill_chunk=64, prefill_budget=budget)
        d = llm.driver
        sids = [d.open([1] + list(range(10 + i, 10 + i + 255)), SamplingParams(max_tokens=200, ignore_eos=True)) for i in range(8)]
        n = 0
        while any(d.seqs[s].generated == 0 for s in sids):
            for r in d.step(sids):
                if r.token is not None:
                    d.commit(r.seq_id, [r.token])
            n += 1
        widest = max(len(x.tokens) for x in llm.driver.engine.steps)
        return n, widest
    one, w1 = steps(None)
    four, w4 = steps(256)
    assert four < one / 3 and w1 <= 64 + 8 and 64 + 8 < w4 <= 256 + 8
