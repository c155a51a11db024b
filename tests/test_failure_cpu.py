"""Failure detection on the host (no GPU, nothing faults): ranks that leave, die or stall; a step that outlives its
deadline; a device wait that gave up.  Every failure is made on the host - a rank that exits or sleeps between steps, a
step engine that sleeps, a status hook that reports a code - and the checks are the contract of the reference's
coordinator on failing devices (crates/poot-executor/tests/coordinator.rs:55-80): the failure is noticed within its
limit, the engine goes dead with a cause, only the live requests fail, nothing hangs."""
import json
import os
import subprocess
import sys
import time

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _group(mode: str, world: int = 2, timeout: int = 240):
    port = 30100 + (os.getpid() % 400) + {"leave": 0, "die": 1, "stall": 2, "instep": 3}[mode] * 401
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "failure_worker.py"), mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    deadline = time.time() + timeout
    for p in procs:
        try:
            out, err = p.communicate(timeout=max(1.0, deadline - time.time()))
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise AssertionError(f"{mode}: a rank did not exit")
        outs.append((p.returncode, out, err))
    return outs


def _leader(outs):
    rc, out, err = outs[0]
    assert rc == 0, err[-3000:]
    return json.loads([l for l in out.splitlines() if l.startswith("{")][-1])


@pytest.mark.parametrize("mode,needle", [("leave", "left the group"), ("die", "no heartbeat"), ("stall", "no readiness")])
def test_leader_notices_a_lost_follower_before_launching_the_step(mode, needle):
    outs = _group(mode)
    lead = _leader(outs)
    assert lead["health"]["status"] == "dead"
    assert "rank 1" in lead["health"]["cause"] and needle in lead["health"]["cause"], lead
    assert lead["finals"] == ["error", "error"] and all("engine fault" in e for e in lead["errors"])
    assert lead["refused_new"]
    assert 0 < min(lead["tokens_before"])            # the group served tokens before the failure
    assert lead["took_s"] < 30
    if mode == "stall":                              # the stalled rank wakes up, sees the stop and leaves by itself
        rc, out, _ = outs[1]
        assert rc == 0 and "RankLost" in json.loads(out.splitlines()[-1])["cause"]
    if mode == "die":
        assert outs[1][0] == 7


def test_a_follower_that_stalls_inside_the_step_ends_the_leaders_collective_with_an_error():
    outs = _group("instep")
    lead = _leader(outs)
    assert lead["health"]["status"] == "dead" and lead["finals"] == ["error", "error"], lead
    assert lead["took_s"] < 40


def _fake_engine_with_jobs(step_deadline=None, engine=None):
    from poot_b200.driver.driver import Driver
    from poot_b200.driver.engines import FakeStepEngine
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.serve.metrics import Metrics
    from poot_b200.serve.scheduler import Job, ServeEngine
    from poot_b200.text.codec import ByteTokenizer
    tk = ByteTokenizer(1000)
    eng = engine or FakeStepEngine(1000, 96)
    drv = Driver(eng, 64, 4, 128, 1000, prefill_chunk=32, eos_token=tk.eos)
    se = ServeEngine(drv, tk, Metrics(), 16, 30.0, step_deadline=step_deadline)
    jobs = [Job(prompt_tokens=[10 + i, 11, 12], params=SamplingParams(max_tokens=50, ignore_eos=True)) for i in range(2)]
    return se, jobs, eng


def test_step_deadline_watchdog_aborts_the_engine_and_fails_live_requests():
    from poot_b200.driver.engines import FakeStepEngine
    from poot_b200.serve.scheduler import EngineDead

    class Slow(FakeStepEngine):
        aborted = 0

        def run_step(self, inp):
            if len(self.steps) == 3:
                t0 = time.time()
                while not self.aborted and time.time() - t0 < 20:      # "a kernel waiting for a peer"
                    time.sleep(0.01)
            return super().run_step(inp)

        def abort(self):
            self.aborted += 1

    se, jobs, eng = _fake_engine_with_jobs(step_deadline=0.5, engine=Slow(1000, 96))
    se.start()
    for j in jobs:
        se.submit(j)
    t0 = time.time()
    finals = [j.wait(timeout=15) for j in jobs]
    assert time.time() - t0 < 10
    assert [f["type"] for f in finals] == ["error", "error"]
    h = se.health()
    assert h["status"] == "dead" and "deadline" in h["cause"]
    assert eng.aborted == 1                           # the abort hook ran: pending device waits were told to give up
    assert se.metrics.to_json()["counters"]["poot_step_deadline_exceeded_total"] == 1
    with pytest.raises(EngineDead):
        se.submit(jobs[0])
    se._stop.set()


def test_a_device_wait_that_gave_up_fails_the_step_and_kills_the_engine():
    """The device engine adapter reads the control block with every step's result.  A non-zero code means the step's
    tokens are invalid: they are not committed, the typed error ends the engine thread, `/health` reports dead."""
    import torch
    from poot_b200 import LLM, SamplingParams
    from poot_b200.ops.cuda_ops import DeviceWaitTimeout
    from poot_b200.serve.metrics import Metrics
    from poot_b200.serve.scheduler import Job, ServeEngine
    from poot_b200.utils.kernel_emulation import emulated_kernels
    with emulated_kernels():
        llm = LLM.random("tiny-llama", device="cpu", rows=2, max_seq=64, prefill_chunk=16, num_blocks=16, std=0.05,
                         vocab=2048, n_layers=2)
        dev = llm.driver.engine.inner          # the device adapter under the lifecycle guard
        calls = {"n": 0}

        def hook():
            calls["n"] += 1
            return (7, 5 * 16 + 1) if calls["n"] == 4 else (0, -1)     # step deadline at site 5 waiting for rank 1
        dev.status_hook = hook
        se = ServeEngine(llm.driver, llm.tokenizer, Metrics(), 16, 30.0)
        se.start()
        job = se.submit(Job(prompt_tokens=[5, 9, 11], params=SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True)))
        final = job.wait(timeout=60)
    assert final["type"] == "error"
    assert len(job.tokens) == 3                      # three good steps were committed, the fourth was discarded
    h = se.health()
    assert h["status"] == "dead" and "step deadline (site 5, waiting for rank 1)" in h["cause"]
    # the adapter raises the typed error itself
    dev.status_hook = lambda: (4, 33)
    with emulated_kernels(), pytest.raises(DeviceWaitTimeout) as err:
        dev._raise_on_failed_wait(False)
    assert err.value.code == 4 and err.value.detail == 33


def test_prefix_cache_evicts_leaves_before_their_parents():
    """Under pressure the cache drops the deepest cached blocks first, so what stays cached can still be matched."""
    from poot_b200.driver.kvcache import BlockPool, PrefixCache
    pool = BlockPool(16)
    cache = PrefixCache(pool)
    toks = np.arange(64, dtype=np.uint32)            # a chain of four full blocks
    blocks = pool.alloc(4)
    cache.register(toks, blocks)
    for b in blocks:                                 # the sequence is released: only the cache holds the blocks
        pool.release(b)
    assert cache.reclaimable() == 4
    assert cache.evict_unused(2) == 2
    got = cache.match(toks)                       # the two blocks nearest the root are still matchable
    assert len(got) == 2 and list(got) == list(blocks[:2])
    for b in got:
        pool.release(b)
    # a block that a live sequence shares is not reclaimable
    held = cache.match(toks[:17])
    assert cache.reclaimable() == 1
    pool.release(held[0])
    assert cache.evict_unused(0) == 2 and len(cache) == 0
