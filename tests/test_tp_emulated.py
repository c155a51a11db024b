"""The fused tensor-parallel programs of the engine with the ranks as threads over host restatements of the kernels
(``utils/tp_emulation.py``): token parity with one rank at world 2, 4 and 8 in both collective forms, the flag targets
across steps, and the failure rules of the waits - host abort, step deadline, poison - driven from the host."""
import threading
import time

import pytest
import torch

from poot_b200.models.config import DecoderConfig
from poot_b200.runtime.engine import DecoderEngine
from poot_b200.runtime.session import FixedBatchSession
from poot_b200.runtime.weights import random_weights
from poot_b200.utils.kernel_emulation import emulated_kernels
from poot_b200.utils.tp_emulation import (ABORTED, PEER_FAILED, STEP_DEADLINE, EmulatedFusedComm, EmulatedGroup)


def _cfg(world):
    return DecoderConfig(n_layers=2, hidden=256, n_heads=8, n_kv_heads=8 if world > 4 else 4, head_dim=64, ffn=512,
                         vocab=4096, max_position=256)


def _prompts(cfg, B=2, P=9):
    g = torch.Generator().manual_seed(5)
    return torch.randint(0, cfg.vocab, (B, P), generator=g, dtype=torch.int32)


def _rank_program(cfg, rank, world, comm, mode, steps, out, before_step=None):
    w = random_weights(cfg, "cpu", seed=0, std=0.05, tp_rank=rank, tp_world=world)
    eng = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=48, max_blocks_per_seq=4, comm=comm, device="cpu",
                        use_graphs=False)
    if mode == "rs_ag":
        eng.tp_mode = "rs_ag"
    s = FixedBatchSession(eng, 2, 64)
    toks = [s.prefill_fast(_prompts(cfg)).clone()]
    for i in range(steps):
        if before_step is not None:
            before_step(rank, i)
        toks.append(s.decode(toks[-1][:, 0].tolist()).clone())
    out[rank] = torch.stack(toks)


def _run_group(cfg, world, mode, steps=3, before_step=None, budget=5.0):
    group = EmulatedGroup(world, cfg.hidden)
    for c in group.ctl:
        c["budget"] = budget
    comms = [EmulatedFusedComm(r, group) for r in range(world)]
    out, errs = {}, {}

    def body(r):
        try:
            _rank_program(cfg, r, world, comms[r], mode, steps, out, before_step)
        except Exception as e:       # a thread's failure must fail the test, not vanish
            errs[r] = e
    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=180)
    assert not any(t.is_alive() for t in threads), "a rank thread did not finish"
    return group, comms, out, errs


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["oneshot", "rs_ag"])
def test_fused_programs_match_one_rank_at_every_world_size(world, mode):
    cfg = _cfg(world)
    with emulated_kernels():
        ref = {}
        _rank_program(cfg, 0, 1, None, "oneshot", 3, ref)
        group, comms, out, errs = _run_group(cfg, world, mode)
    assert not errs, errs
    for r in range(world):
        assert torch.equal(out[r][:, :, 0], ref[0][:, :, 0]), (r, out[r][:, :, 0], ref[0][:, :, 0])
        assert group.status(r) == (0, -1)
    # one epoch per step; flag targets never repeat and grow by one per site inside a step
    L = cfg.n_layers
    assert all(c.epoch == 4 for c in comms)
    rs_targets = [t for k, _, t in comms[0].log if k == "rs"]
    assert rs_targets == sorted(set(rs_targets)) and len(rs_targets) == 4 * 2 * L
    assert rs_targets[-1] == 4 * 2 * L
    if mode == "rs_ag":                              # the 18-token prefill and the decode steps both ride the sharded form
        ag_targets = [t for k, _, t in comms[0].log if k == "ag"]
        assert len(ag_targets) == 4 * (2 * L + 1) and ag_targets == sorted(set(ag_targets))
    assert all(c.ax_count == 4 for c in comms)       # one greedy-pick exchange per step, no library collective


def test_host_abort_ends_a_pending_wait_at_once():
    """Rank 1 never starts its second decode step.  Rank 0 sits in a wait with a long budget; the host sets the abort
    word and the wait returns within milliseconds, the first cause says so, and later waits do not wait at all."""
    cfg = _cfg(2)
    gate = threading.Event()
    holder = {}

    def before(rank, i):
        if rank == 1 and i == 1:
            gate.wait(timeout=30)                     # stays out of the step until the test lets it go

    def aborter():
        time.sleep(0.5)
        holder["t_abort"] = time.monotonic()
        holder["group"].request_abort(0)
        time.sleep(0.3)
        holder["group"].request_abort(1)
        gate.set()

    with emulated_kernels():
        group = EmulatedGroup(2, cfg.hidden)
        for c in group.ctl:
            c["budget"] = 60.0
        holder["group"] = group
        comms = [EmulatedFusedComm(r, group) for r in range(2)]
        out = {}
        ts = [threading.Thread(target=_rank_program, args=(cfg, r, 2, comms[r], "oneshot", 3, out, before), daemon=True)
              for r in range(2)]
        threading.Thread(target=aborter, daemon=True).start()
        t0 = time.monotonic()
        for t in ts:
            t.start()
        ts[0].join(timeout=60)
        done0 = time.monotonic()
        ts[1].join(timeout=60)
    assert not ts[0].is_alive() and not ts[1].is_alive()
    assert done0 - holder["t_abort"] < 2.0            # not the 60 s budget
    code, detail = group.status(0)
    assert code == ABORTED and detail % 16 == 1       # it was waiting for rank 1
    assert group.ctl[0]["gave_up"] >= 1


def test_the_waits_of_one_step_share_one_deadline_and_the_failure_reaches_the_peer():
    """Rank 1 stalls for longer than the step budget before its second decode step.  Rank 0 gives up at the deadline
    (once: the later waits of the step return at once), publishes its failure with its next signal, and rank 1, when it
    finally runs the step, stops waiting as soon as it sees the poison word."""
    cfg = _cfg(2)

    def before(rank, i):
        if rank == 1 and i == 1:
            time.sleep(1.2)

    with emulated_kernels():
        t0 = time.monotonic()
        group, comms, out, errs = _run_group(cfg, 2, "oneshot", steps=2, before_step=before, budget=0.4)
        took = time.monotonic() - t0
    assert not errs, errs
    assert group.status(0)[0] == STEP_DEADLINE
    assert group.status(1)[0] in (PEER_FAILED, STEP_DEADLINE)
    assert group.ctl[0]["gave_up"] <= 2 * cfg.n_layers + 2
    assert took < 10.0                                # one budget, not one per site


def test_device_adapter_turns_the_emulated_status_into_a_typed_error():
    from poot_b200.driver.engines import DeviceStepEngine
    from poot_b200.ops.cuda_ops import DeviceWaitTimeout
    cfg = _cfg(2)
    with emulated_kernels():
        group = EmulatedGroup(2, cfg.hidden)
        w = random_weights(cfg, "cpu", seed=0, std=0.05, tp_rank=0, tp_world=2)
        eng = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=48, max_blocks_per_seq=4,
                            comm=EmulatedFusedComm(0, group), device="cpu", use_graphs=False)
        dev = DeviceStepEngine(eng)
        dev.status_hook = lambda: group.status(0)
        group.fail(0, STEP_DEADLINE, 3 * 16 + 1)
        with pytest.raises(DeviceWaitTimeout, match=r"step deadline \(site 3, waiting for rank 1\)"):
            dev._raise_on_failed_wait(False)


def _moe_rank_program(cfg, rank, world, comm, steps, out):
    w = random_weights(cfg, "cpu", seed=0, std=0.05, tp_rank=rank, tp_world=world, ep_rank=rank, ep_world=world)
    eng = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=48, max_blocks_per_seq=4, comm=comm, device="cpu",
                        use_graphs=False)
    s = FixedBatchSession(eng, 2, 64)
    toks = [s.prefill_fast(_prompts(cfg)).clone()]
    for _ in range(steps):
        toks.append(s.decode(toks[-1][:, 0].tolist()).clone())
    out[rank] = torch.stack(toks)
    return eng


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_steps_are_fused_for_one_or_several_experts_per_rank(world):
    """Four routed experts over 2 ranks (two per rank: the combine kernel pushes) and over 4 ranks (one per rank: the
    down projection's epilogue pushes): tokens equal the single-rank run, and no step used a library collective."""
    cfg = DecoderConfig(n_layers=2, hidden=256, n_heads=8, n_kv_heads=4, head_dim=64, ffn=512, vocab=4096, max_position=256,
                        n_experts=4, top_k=2, moe_ffn=128)
    with emulated_kernels():
        ref = {}
        _moe_rank_program(cfg, 0, 1, None, 3, ref)
        group = EmulatedGroup(world, cfg.hidden)
        for c in group.ctl:
            c["budget"] = 5.0
        comms = [EmulatedFusedComm(r, group) for r in range(world)]
        out, errs = {}, {}

        def body(r):
            try:
                _moe_rank_program(cfg, r, world, comms[r], 3, out)
            except Exception as e:
                errs[r] = e
        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=180)
        assert not any(t.is_alive() for t in threads), "a rank thread did not finish"
    assert not errs, errs
    for r in range(world):
        # every rank reduces the same inbox rows in the same order: the ranks agree bit for bit with one another ...
        assert torch.equal(out[r], out[0]) and group.status(r) == (0, -1)
    # ... and with one rank up to the rounding of the per-rank partial sums (bf16 partials added in rank order instead
    # of one f32 sum over the token's experts): the prompt's token and the first decoded token are the same
    assert torch.equal(out[0][:2, :, 0], ref[0][:2, :, 0]), (out[0][:, :, 0], ref[0][:, :, 0])
    assert (out[0][:, :, 0] == ref[0][:, :, 0]).float().mean() >= 0.75
    L = cfg.n_layers
    rs_targets = [t for k, _, t in comms[0].log if k == "rs"]
    assert len(rs_targets) == 4 * 2 * L and rs_targets == sorted(set(rs_targets))     # attention + experts, every step
    assert all(c.ax_count == 4 for c in comms) and all(c.library_collectives == 0 for c in comms)


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_dispatch_and_combine_over_a_token_sharded_stream(world):
    """The reduce-scatter form with routed experts: each rank normalises its own token rows, dispatches every
    (token, slot) row to the rank of its expert, runs its experts over what it received and sends the rows back; the
    owner sums.  Tokens follow the single-rank run, every rank agrees with every other, no library collective is used,
    and a row only travels to the ranks of its experts."""
    cfg = DecoderConfig(n_layers=2, hidden=256, n_heads=8, n_kv_heads=4, head_dim=64, ffn=512, vocab=4096, max_position=256,
                        n_experts=8, top_k=2, moe_ffn=128)
    with emulated_kernels():
        ref = {}
        _moe_rank_program(cfg, 0, 1, None, 3, ref)
        group = EmulatedGroup(world, cfg.hidden)
        for c in group.ctl:
            c["budget"] = 5.0
        comms = [EmulatedFusedComm(r, group) for r in range(world)]
        out, errs, engines = {}, {}, {}

        def body(r):
            try:
                w = random_weights(cfg, "cpu", seed=0, std=0.05, tp_rank=r, tp_world=world, ep_rank=r, ep_world=world)
                eng = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=48, max_blocks_per_seq=4, comm=comms[r],
                                    device="cpu", use_graphs=False)
                eng.tp_mode = "rs_ag"
                engines[r] = eng
                s = FixedBatchSession(eng, 2, 64)
                toks = [s.prefill_fast(_prompts(cfg)).clone()]
                for _ in range(3):
                    toks.append(s.decode(toks[-1][:, 0].tolist()).clone())
                out[r] = torch.stack(toks)
            except Exception as e:
                errs[r] = e
        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=240)
        assert not any(t.is_alive() for t in threads), "a rank thread did not finish"
    assert not errs, errs
    for r in range(world):
        assert torch.equal(out[r], out[0]) and group.status(r) == (0, -1)
    # bf16 partial sums of the sharded attention move the router's inputs by an ulp, which can flip a near-tie of two
    # experts; the layer itself is checked bit for bit below.  Here: the prompt's tokens agree, most later ones do
    assert torch.equal(out[0][0, :, 0], ref[0][0, :, 0]), (out[0][:, :, 0], ref[0][:, :, 0])
    assert (out[0][:, :, 0] == ref[0][:, :, 0]).float().mean() >= 0.5
    L = cfg.n_layers
    kinds = [k for k, _, _ in comms[0].log]
    assert kinds.count("epd") == 4 * L and kinds.count("epc") == 4 * L          # one dispatch and one combine per routed layer
    assert kinds.count("rs") == 4 * L                                            # only the attention output is reduce-scattered
    assert all(c.library_collectives == 0 for c in comms)
    # a rank's receive counts sum to the (token, slot) rows of the whole step: nothing was sent twice
    par = comms[0]._ep_target(L - 1) & 1
    total = sum(int(group.ep_count[d][par, s]) for d in range(world) for s in range(world))
    S = comms[0].rows_for(2) // world
    assert total == world * S * cfg.top_k


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_expert_layer_equals_the_single_rank_layer_bit_for_bit(world):
    """Same normalised rows in, same routing: dispatch, grouped experts on the owning ranks and combine give exactly what
    one rank computes over all rows (each (token, slot) row is one expert's product whichever rank runs it, and the
    owner adds a token's rows in slot order)."""
    from poot_b200.runtime import moe as MOE
    cfg = DecoderConfig(n_layers=1, hidden=256, n_heads=8, n_kv_heads=4, head_dim=64, ffn=512, vocab=4096, max_position=256,
                        n_experts=8, top_k=2, moe_ffn=128)
    S = 8
    X = (torch.randn(world * S, 256, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16)
    with emulated_kernels():
        w = random_weights(cfg, "cpu", seed=0, std=0.05)
        one = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=64, max_blocks_per_seq=4, device="cpu", use_graphs=False)
        want = torch.zeros(world * S, 256, dtype=torch.bfloat16)
        MOE.moe_forward(one, 0, w.layers[0], X.clone(), world * S, None, h=want)
        group = EmulatedGroup(world, cfg.hidden)
        comms = [EmulatedFusedComm(r, group) for r in range(world)]
        got, errs = {}, {}

        def body(r):
            try:
                wr = random_weights(cfg, "cpu", seed=0, std=0.05, tp_rank=r, tp_world=world, ep_rank=r, ep_world=world)
                eng = DecoderEngine(wr, num_blocks=9, max_seqs=2, max_tokens=64, max_blocks_per_seq=4, comm=comms[r],
                                    device="cpu", use_graphs=False)
                for _ in range(2):                      # two exchanges: both parities of the receive and combine areas
                    comms[r].begin_step()
                    comms[r].h_shard[:S].zero_()
                    MOE.moe_forward_sharded(eng, 0, wr.layers[0], X[r * S:(r + 1) * S].clone(), S, comms[r], site=0)
                got[r] = comms[r].h_shard[:S].clone()
            except Exception as e:
                errs[r] = e
        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=120)
    assert not errs, errs
    assert torch.equal(torch.cat([got[r] for r in range(world)], 0), want)
    assert want.float().abs().max().item() > 0.05


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("moe", [False, True])
def test_prefill_sized_steps_ride_the_sharded_program(world, moe):
    """A 200-token prefill (256 padded rows, 128 or 64 per rank) goes through the token-sharded program - tiled GEMMs with
    the gathered operand and the scattered result on the device, the expert exchange when the model is routed - and the
    decode steps after it through the skinny ones; no library collective in any step."""
    extra = dict(n_experts=8, top_k=2, moe_ffn=128) if moe else {}
    cfg = DecoderConfig(n_layers=2, hidden=256, n_heads=8, n_kv_heads=4, head_dim=64, ffn=512, vocab=4096, max_position=256,
                        **extra)
    g = torch.Generator().manual_seed(11)
    prompts = torch.randint(0, cfg.vocab, (2, 100), generator=g, dtype=torch.int32)

    def program(rank, w_world, comm, out):
        w = random_weights(cfg, "cpu", seed=0, std=0.05, tp_rank=rank, tp_world=w_world,
                           **(dict(ep_rank=rank, ep_world=w_world) if moe else {}))
        eng = DecoderEngine(w, num_blocks=20, max_seqs=2, max_tokens=256, max_blocks_per_seq=8, comm=comm, device="cpu",
                            use_graphs=False)
        eng.tp_mode = "rs_ag"
        s = FixedBatchSession(eng, 2, 128)
        toks = [s.prefill_fast(prompts).clone()]
        toks.append(s.decode(toks[-1][:, 0].tolist()).clone())
        out[rank] = (torch.stack(toks), eng)

    with emulated_kernels():
        ref = {}
        program(0, 1, None, ref)
        group = EmulatedGroup(world, cfg.hidden, max_rows=256)
        for c in group.ctl:
            c["budget"] = 20.0
        comms = [EmulatedFusedComm(r, group) for r in range(world)]
        out, errs = {}, {}

        def body(r):
            try:
                program(r, world, comms[r], out)
            except Exception as e:
                errs[r] = e
        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=300)
        assert not any(t.is_alive() for t in threads), "a rank thread did not finish"
    assert not errs, errs
    assert comms[0].rows_for(200) == 256 and comms[0].s_max == 256 // world
    for r in range(world):
        assert torch.equal(out[r][0], out[0][0]) and group.status(r) == (0, -1)
        assert comms[r].library_collectives == 0
    assert torch.equal(out[0][0][0, :, 0], ref[0][0][0, :, 0]), (out[0][0][:, :, 0], ref[0][0][:, :, 0])
    kinds = [k for k, _, _ in comms[0].log]
    L = cfg.n_layers
    assert kinds.count("ag") == 2 * ((L + 1) if moe else (2 * L + 1))        # gathers: per attention (+ per dense FFN) + the head
    assert kinds.count("epd") == (2 * L if moe else 0)
