"""The step engine's failure lifecycle on fake engines with injected failures: validation before launch, NeedsReset
after a failed transaction, exactly one abort per failure, Poisoned when the clean-up or the reset fails too
(the contract of crates/poot-executor/src/error.rs:12-57 as tested in crates/poot-executor/tests/coordinator.rs:55-80)."""
import numpy as np
import pytest

from poot_b200.driver.driver import Driver
from poot_b200.driver.engines import FakeStepEngine
from poot_b200.driver.sampler import SamplingParams
from poot_b200.runtime.lifecycle import (Fault, GuardedStepEngine, NeedsReset, Poisoned, StepLimits, Validation,
                                         validate_step)


class Flaky(FakeStepEngine):
    """Fails the step numbered ``fail_at_step``; counts clean-ups and resets; either can be made to fail."""

    def __init__(self, *a, cleanup_fails=False, reset_fails=False, **kw):
        super().__init__(*a, **kw)
        self.cleanups = self.resets = 0
        self.cleanup_fails, self.reset_fails = cleanup_fails, reset_fails

    def abort_cleanup(self):
        self.cleanups += 1
        if self.cleanup_fails:
            raise RuntimeError("injected: the device did not go idle")

    def reset_state(self):
        self.resets += 1
        if self.reset_fails:
            raise RuntimeError("injected: reset failed")
        self.fail_at_step = None


def _driver(engine):
    return Driver(engine, 64, 4, 128, 1000, prefill_chunk=32, eos_token=None)


def test_a_failed_step_needs_a_complete_reset_before_the_next_one():
    eng = Flaky(1000, 96, fail_at_step=2)
    d = _driver(eng)
    assert isinstance(d.engine, GuardedStepEngine) and d.engine.state == "ready"
    sid = d.open([5, 6, 7], SamplingParams(max_tokens=20, ignore_eos=True))
    for _ in range(2):
        (r,) = d.step([sid])
        d.commit(sid, [r.token])
    with pytest.raises(Fault, match="injected engine fault"):
        d.step([sid])
    assert d.engine.state == "needs_reset" and eng.cleanups == 1 and d.engine.aborts == 1
    with pytest.raises(NeedsReset):                  # refused until the reset, and no second abort
        d.step([sid])
    with pytest.raises(NeedsReset):
        d.engine.write_block_table(0, [1, 2])
    assert eng.cleanups == 1
    blocks_held = d.pool.num_blocks - d.pool.available
    assert blocks_held > 0
    d.reset()                                        # complete: engine state, sequences, blocks, prefix cache
    assert d.engine.state == "ready" and eng.resets == 1
    assert not d.seqs and d.pool.available == d.pool.num_blocks and len(d._free_rows) == 4
    assert d.generate([5, 6, 7], SamplingParams(max_tokens=3, ignore_eos=True)) == [8, 9, 10]


def test_a_failing_cleanup_poisons_the_engine_for_good():
    eng = Flaky(1000, 96, fail_at_step=0, cleanup_fails=True)
    d = _driver(eng)
    sid = d.open([1, 2, 3])
    with pytest.raises(Fault):
        d.step([sid])
    assert d.engine.state == "poisoned"
    with pytest.raises(Poisoned):
        d.step([sid])
    with pytest.raises(Poisoned):                    # a reset cannot clear it
        d.reset()
    assert eng.resets == 0 and eng.cleanups == 1


def test_a_failing_reset_poisons_too():
    eng = Flaky(1000, 96, fail_at_step=0, reset_fails=True)
    d = _driver(eng)
    sid = d.open([1, 2, 3])
    with pytest.raises(Fault):
        d.step([sid])
    assert d.engine.state == "needs_reset"
    with pytest.raises(Poisoned, match="reset failed"):
        d.reset()
    with pytest.raises(Poisoned):
        d.step([sid])


def test_validation_refuses_before_launch_and_leaves_the_engine_ready():
    eng = Flaky(1000, 96)
    d = _driver(eng)
    sid = d.open([1, 2, 3], SamplingParams(max_tokens=4, ignore_eos=True))
    inp = d.build_inputs(d.plan([sid]))
    lim = StepLimits(vocab=1000, max_tokens=96, max_rows=4, pool_slots=64 * 16, max_position=128)
    validate_step(inp, lim)                          # the planned step is in range
    d.engine.limits = lim
    for field, value, needle in (("tokens", 1000, "token id"), ("slots", 64 * 16, "K/V slot"),
                                 ("positions", 128, "position"), ("logit_idx", len(inp.tokens), "logit row")):
        broken = d.build_inputs(d.plan([sid]))
        getattr(broken, field)[0] = value
        with pytest.raises(Validation, match=needle):
            d.engine.run_step(broken)
        assert d.engine.state == "ready" and len(eng.steps) == 0 and eng.cleanups == 0     # nothing ran, nothing to clean
    (r,) = d.step([sid])                             # and the engine still serves
    assert r.token == 4


def test_kernel_reported_failure_keeps_its_code():
    from poot_b200.ops.cuda_ops import DeviceWaitTimeout

    class Timeout(Flaky):
        def run_step(self, inp):
            raise DeviceWaitTimeout("device wait timed out in peer flag (site 3, waiting for rank 2)", 4, 3 * 16 + 2)

    d = _driver(Timeout(1000, 96))
    sid = d.open([1, 2, 3])
    with pytest.raises(Fault) as err:
        d.step([sid])
    assert err.value.code == 4 and err.value.detail == 50
    assert isinstance(err.value.__cause__, DeviceWaitTimeout)
