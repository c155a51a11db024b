"""Feature table, placement rules, capacity fit, speculative decoding and beam search on the host engine."""
import numpy as np
import pytest

from poot_b200.driver import capacity
from poot_b200.driver.beam import beam_search, fork
from poot_b200.driver.features import Feature, Incompatible, Unavailable, check
from poot_b200.driver.placement import Placement, PlacementError
from poot_b200.driver.sampler import SamplingParams
from poot_b200.driver.speculate import LookupDraft, ModelDraft, generate_speculative
from poot_b200.llm import LLM
from poot_b200.models.config import llama3_8b, llama3_70b, mixtral_8x7b


def test_feature_table():
    check([Feature.TENSOR_PLACEMENT, Feature.PREFIX_CACHE, Feature.LOGPROBS, Feature.GUIDED])
    with pytest.raises(Incompatible) as e:
        check([Feature.BEAM, Feature.TENSOR_PLACEMENT])
    assert "vocabulary" in str(e.value)
    with pytest.raises(Incompatible):
        check([Feature.DRAFT_LOOKUP, Feature.GUIDED])
    check([Feature.RECURRENT_STATE, Feature.GUIDED, Feature.LOGPROBS])       # recurrent families serve; what they exclude is typed
    for other in (Feature.PREFIX_CACHE, Feature.BEAM):
        with pytest.raises(Incompatible):
            check([Feature.RECURRENT_STATE, other])
    check([Feature.RECURRENT_STATE, Feature.DRAFT_LOOKUP])       # the round snapshots and restores the state rows
    with pytest.raises(Incompatible):
        check([Feature.ADAPTERS, Feature.TENSOR_PLACEMENT])
    check([Feature.DRAFT_MTP])                   # offered; a model without the layer is refused where the model is known
    with pytest.raises(Unavailable):
        from poot_b200.driver.features import require_mtp
        from poot_b200.models.config import tiny_llama
        require_mtp(tiny_llama())
    check([Feature.EXPERT_POOL, Feature.PREFIX_CACHE])
    with pytest.raises(Incompatible):
        check([Feature.EXPERT_POOL, Feature.EXPERT_PLACEMENT])


def test_placement_parse_and_divisibility():
    p = Placement.parse("tensor:0,1,2,3")
    assert p.kind == "tensor" and p.world == 4 and p.features == [Feature.TENSOR_PLACEMENT]
    p.validate(llama3_8b())
    Placement.parse("tensor:0,1,2,3,4,5,6,7").validate(llama3_70b())
    Placement.parse("expert:0,1,2,3,4,5,6,7").validate(mixtral_8x7b())
    for bad in ("tensor", "tensor:a", "tensor:0,0", "tensor:0,1,2", "ring:0,1"):
        with pytest.raises(PlacementError):
            Placement.parse(bad)
    pp = Placement.parse("pipeline:0,1,2")
    assert pp.kind == "pipeline" and pp.world == 3 and pp.features == [Feature.PIPELINE_PLACEMENT]
    pp.validate(llama3_8b())
    from poot_b200.driver.placement import pipeline_cuts
    cuts = pipeline_cuts(llama3_70b(), 8)
    assert cuts[0][0] == 0 and cuts[-1][1] == 80 and all(a < b for a, b in cuts) and all(cuts[i][1] == cuts[i + 1][0] for i in range(7))
    # the embedding sits on the first stage and the head on the last: they carry fewer layers than the middle stages
    sizes = [b - a for a, b in cuts]
    assert sizes[0] < max(sizes) and sizes[-1] < max(sizes) and max(sizes) - min(sizes) <= 2
    with pytest.raises(Incompatible):
        check([Feature.PIPELINE_PLACEMENT, Feature.TENSOR_PLACEMENT])
    with pytest.raises(PlacementError):
        Placement.parse("expert:0,1").validate(llama3_8b())
    with pytest.raises(PlacementError):
        Placement.parse("tensor:" + ",".join(map(str, range(16)))).validate(llama3_8b().__class__(**{**vars(llama3_8b()), "n_heads": 24}))


def test_capacity_fit_halves_until_it_fits():
    cfg = llama3_8b()
    big = capacity.fit(cfg, free_bytes=150 << 30, rows=64, max_seq=8192)
    assert (big.rows, big.max_seq) == (64, 8192) and big.num_blocks == 64 * 512 + 1
    assert big.kv_bytes == big.num_blocks * capacity.kv_bytes_per_block(cfg) == big.num_blocks * 32 * 2 * 8 * 16 * 128 * 2
    small = capacity.fit(cfg, free_bytes=1 << 30, rows=64, max_seq=8192)
    assert small.max_seq < 8192 and small.rows == 64         # one full-length sequence must fit: the length is halved
    assert small.planned_bytes <= (1 << 30) - capacity.RESERVE
    assert small.num_blocks >= capacity.blocks_for(small.max_seq) + 1
    tp = capacity.fit(cfg, free_bytes=1 << 30, rows=64, max_seq=8192, tp_world=8)
    assert tp.max_seq == 8192 and tp.num_blocks > small.num_blocks      # a rank holds 1/8 of the KV heads
    with pytest.raises(capacity.DoesNotFit):
        capacity.fit(cfg, free_bytes=300 << 20, rows=4, max_seq=4096)
    assert capacity.candidates(8, 512) == [(8, 512), (8, 256), (8, 128), (4, 128), (2, 128), (1, 128)]


def test_lookup_drafting_equals_plain_greedy_with_fewer_steps():
    prompt = [1] + list(range(3, 49)) + [3, 4, 5]
    plain = LLM.fake(vocab=50).driver
    ref = plain.generate(prompt, SamplingParams(max_tokens=30, ignore_eos=True))
    d = LLM.fake(vocab=50).driver
    got = generate_speculative(d, prompt, SamplingParams(max_tokens=30, ignore_eos=True), LookupDraft.parse("3:4"))
    assert got == ref
    assert d.stats["steps"] < plain.stats["steps"] / 2 and d.stats["draft_accepted"] > 0
    assert d.kv_usage()["blocks_used"] == d.kv_usage()["prefix_entries"]
    with pytest.raises(ValueError):
        LookupDraft.parse("3")


def test_rejected_drafts_do_not_change_the_output():
    class WrongDraft:
        def propose(self, tokens):
            return [7, 7, 7]
    prompt = [1, 10, 11, 12]
    ref = LLM.fake(vocab=50).driver.generate(prompt, SamplingParams(max_tokens=12, ignore_eos=True))
    d = LLM.fake(vocab=50).driver
    assert generate_speculative(d, prompt, SamplingParams(max_tokens=12, ignore_eos=True), WrongDraft()) == ref
    assert d.stats["draft_accepted"] <= 1 and d.stats["draft_proposed"] > 0


def test_model_drafting_with_a_second_driver():
    prompt = [1, 20, 21]
    ref = LLM.fake(vocab=60).driver.generate(prompt, SamplingParams(max_tokens=10, ignore_eos=True))
    d = LLM.fake(vocab=60).driver
    got = generate_speculative(d, prompt, SamplingParams(max_tokens=10, ignore_eos=True), ModelDraft(LLM.fake(vocab=60).driver, 3))
    assert got == ref and d.stats["draft_accepted"] >= 6


def test_fork_shares_full_blocks_and_copies_the_partial_one():
    llm = LLM.fake(vocab=100)
    d = llm.driver
    sid = d.open([1] + list(range(3, 23)), SamplingParams(max_tokens=8, ignore_eos=True))   # 21 tokens: 1 full block + 5
    d.step([sid])
    child = fork(d, sid)
    a, b = d.seqs[sid], d.seqs[child]
    assert a.blocks[0] == b.blocks[0] and d.pool.refcount(a.blocks[0]) == 3      # two sequences + the prefix cache
    assert a.blocks[1] != b.blocks[1] and d.engine.copies == [(a.blocks[1], b.blocks[1])]
    assert a.row != b.row and b.tokens == a.tokens and b.computed == a.computed
    d.release(sid, "preempted"); d.release(child, "preempted")
    assert d.kv_usage()["blocks_used"] == d.kv_usage()["prefix_entries"] == 1


def test_fork_carries_the_adapter_the_embedding_rows_and_the_rotary_offset():
    import numpy as np
    d = LLM.fake(vocab=100).driver
    prompt = [1] + list(range(3, 23))
    rope = np.stack([np.arange(21), np.arange(21), np.arange(21)]).astype(np.int32)
    rope[:, 5:] += 7                                          # an image earlier in the prompt pushed the positions on
    sid = d.open(prompt, SamplingParams(max_tokens=4, ignore_eos=True), adapter_slot=2,
                 embeds=(np.array([2, 3]), np.ones((2, 8), np.float32)), rope_positions=rope)
    d.step([sid])
    child = fork(d, sid)
    a, b = d.seqs[sid], d.seqs[child]
    assert b.adapter_slot == 2 and b.rope_delta == a.rope_delta == 7 and b.embed_pos is a.embed_pos and b.identity == a.identity
    d.commit(child, [50])
    inp = d.build_inputs(d.plan([child]))
    assert inp.rope_positions[:, 0].tolist() == [21 + 7] * 3 and inp.adapter_rows[0] == 2 and inp.embed_flags is None
    d.release(sid, "preempted"); d.release(child, "preempted")


def test_beam_search_orders_hypotheses_by_score():
    d = LLM.fake(vocab=40, rows=8).driver
    beams = beam_search(d, [1, 10], width=3, max_tokens=4, eos=-1)
    assert len(beams) == 3
    # the host engine's logits favour last+1, then last+2, ... half a nat apart: the best beam is the +1 chain
    assert beams[0].tokens == [11, 12, 13, 14]
    scores = [b.score for b in beams]
    assert scores == sorted(scores, reverse=True) and scores[0] > scores[1]
    assert beams[1].tokens != beams[0].tokens and len(set(map(lambda b: tuple(b.tokens), beams))) == 3
    assert not d.seqs and d.kv_usage()["blocks_used"] == d.kv_usage()["prefix_entries"]


def test_speculation_on_a_recurrent_hybrid_rolls_its_state_back():
    """A model with gated-delta-net layers: a rejected draft has been folded into the recurrent state, so the verify
    round snapshots the sequence's state rows, restores them after a partial accept and replays the kept tokens; the
    output equals plain greedy decoding token for token."""
    import numpy as np
    import torch
    from poot_b200.driver.driver import Driver
    from poot_b200.driver.engines import DeviceStepEngine
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.driver.speculate import generate_speculative
    from poot_b200.models.registry import Registry
    from poot_b200.oracle.runner import random_weights_f32
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import from_named_tensors
    from poot_b200.utils.kernel_emulation import emulated_kernels
    from test_engine_emulated import HF_BASE, HF_FAMILIES
    model = Registry.builtin().resolve_hf({**HF_BASE, **HF_FAMILIES["qwen3_5"]})
    cfg = model.cfg
    w = random_weights_f32(model, seed=2, std=0.08)
    for k in w:
        if k.endswith("gdn_a_log"):
            w[k] = np.log(np.random.default_rng(3).uniform(0.5, 4.0, w[k].shape)).astype(np.float32)
    named = {k: torch.from_numpy(v).to(torch.bfloat16).float() for k, v in w.items()}

    class Wrong:
        """Drafts that are right for one token and then wrong: every round is a partial accept."""

        def __init__(self, truth):
            self.truth, self.n = truth, 0

        def propose(self, tokens):
            done = len(tokens) - 6
            nxt = self.truth[done:done + 1]
            self.n += 1
            return list(nxt) + [(nxt[0] + 1) % cfg.vocab if nxt else 0, 3] if nxt else []

    prompt = [5, 9, 11, 200, 17, 3]
    sp = SamplingParams(max_tokens=9, temperature=0.0, ignore_eos=True)
    with emulated_kernels():
        def driver():
            eng = DecoderEngine(from_named_tensors(cfg, named, "cpu"), num_blocks=8, max_seqs=4, max_tokens=32,
                                max_blocks_per_seq=4, device="cpu", use_graphs=False)
            return Driver(DeviceStepEngine(eng), 8, 4, 64, cfg.vocab, prefill_chunk=16, prefix_caching=False)
        want = driver().generate(prompt, sp)
        d = driver()
        assert d.engine.has_recurrent_state
        got = generate_speculative(d, prompt, sp, Wrong(want))
    assert got == want
    assert d.stats["draft_replays"] >= 2 and d.stats["draft_accepted"] >= 2


def test_expert_residency_manager_follows_the_lru_contract():
    from poot_b200.driver.expert_residency import ExpertIdOutOfRange, ExpertResidency, PoolTooSmall
    m = ExpertResidency()
    fills, emap, changed = m.sync("L0", [3, 1, 3], experts=8, slots=3)
    assert fills == [(0, 3), (1, 1)] and emap == [-1, 1, -1, 0, -1, -1, -1, -1] and changed     # free rows first
    fills, emap, changed = m.sync("L0", [1, 3], 8, 3)
    assert fills == [] and not changed                                                          # all hits
    fills, _, _ = m.sync("L0", [5], 8, 3)
    assert fills == [(2, 5)]
    fills, emap, _ = m.sync("L0", [1, 7], 8, 3)        # 1 is pinned; 3 was needed least recently of the unpinned rows
    assert fills == [(0, 7)] and emap[3] == -1 and emap[7] == 0 and emap[1] == 1
    assert m.counters.refills == 4 and m.counters.evictions == 1 and m.counters.syncs == 4 and m.counters.id_reads == 8
    _, other, _ = m.sync("L1", [0], 8, 3)              # another layer has its own LRU
    assert other[0] == 0
    with pytest.raises(PoolTooSmall):
        m.sync("L0", [0, 1, 2, 3], 8, 3)
    with pytest.raises(ExpertIdOutOfRange):
        m.sync("L0", [8], 8, 3)
    m.reset()
    assert m.counters.syncs == 0 and not m.sites


def test_pooled_experts_generate_what_resident_experts_generate():
    """Six resident experts of eight per layer, the rest in host memory: the routed layers are cut at the router, the
    manager refills pool rows, and the tokens equal the engine that keeps every expert on the device."""
    import torch
    from poot_b200.driver.expert_residency import ExpertResidency
    from poot_b200.models.config import DecoderConfig
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    from poot_b200.utils.kernel_emulation import emulated_kernels
    cfg = DecoderConfig(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512, max_position=256,
                        n_experts=8, top_k=2, moe_ffn=64)
    prompts = torch.randint(0, cfg.vocab, (1, 3), generator=torch.Generator().manual_seed(4), dtype=torch.int32)

    def run(pool):
        eng = DecoderEngine(random_weights(cfg, "cpu", seed=1, std=0.05), num_blocks=8, max_seqs=1, max_tokens=32,
                            max_blocks_per_seq=4, device="cpu", use_graphs=False)
        mgr = None
        if pool:
            mgr = ExpertResidency()
            eng.enable_expert_pool(pool, mgr)
            assert eng.w.layers[0].ex_wgu.shape[0] == pool and eng.w.layers[0].ex_host[0].shape[0] == 8
        s = FixedBatchSession(eng, 1, 64)
        out = [s.prefill_fast(prompts).clone()]
        for _ in range(12):
            out.append(s.decode(out[-1][:, 0].tolist()).clone())
        return torch.stack(out), mgr

    with emulated_kernels():
        want, _ = run(0)
        got, mgr = run(6)
    assert torch.equal(got, want)
    c = mgr.counters
    assert c.syncs == 13 * cfg.n_layers and c.refills >= 6 and c.refill_bytes > 0
    with emulated_kernels(), pytest.raises(ValueError):
        eng = DecoderEngine(random_weights(cfg, "cpu", seed=1, std=0.05), num_blocks=8, max_seqs=1, max_tokens=32,
                            max_blocks_per_seq=4, device="cpu", use_graphs=False)
        eng.enable_expert_pool(8, ExpertResidency())             # not smaller than the experts


def test_hosted_embedding_rows_are_copied_at_bind_and_change_nothing():
    """The token-embedding table in host memory: bind copies the rows a step gathers into a device slot; tokens equal."""
    import torch
    from poot_b200.models.config import DecoderConfig
    from poot_b200.runtime.engine import DecoderEngine, StepShape
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    from poot_b200.utils.kernel_emulation import emulated_kernels
    cfg = DecoderConfig(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512, max_position=256)
    prompts = torch.randint(0, cfg.vocab, (2, 11), generator=torch.Generator().manual_seed(4), dtype=torch.int32)

    def run(hosted):
        eng = DecoderEngine(random_weights(cfg, "cpu", seed=1, std=0.05), num_blocks=16, max_seqs=2, max_tokens=32,
                            max_blocks_per_seq=4, device="cpu", use_graphs=False)
        freed = eng.host_embedding() if hosted else 0
        s = FixedBatchSession(eng, 2, 64)
        out = [s.prefill_fast(prompts).clone()]
        for _ in range(4):
            out.append(s.decode(out[-1][:, 0].tolist()).clone())
        return torch.stack(out), eng, freed

    with emulated_kernels():
        want, _, _ = run(False)
        got, eng, freed = run(True)
        assert torch.equal(got, want)
        assert freed == cfg.vocab * cfg.hidden * 2 and eng.w.embed.shape == (32, cfg.hidden)      # the device holds a slot, not the table
        with pytest.raises(ValueError, match="chained decode"):
            eng.forward(StepShape(2, 2, 0, chain=True))
        tied = DecoderEngine(random_weights(DecoderConfig(**{**cfg.__dict__, "tie_embeddings": True}), "cpu", seed=1), num_blocks=4,
                             max_seqs=1, max_tokens=16, max_blocks_per_seq=2, device="cpu", use_graphs=False)
        with pytest.raises(ValueError, match="output head"):
            tied.host_embedding()
