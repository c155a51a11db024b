"""The tiny Llama configuration end to end on the CPU oracle: f32 weights ~N(0, 0.02) from seed 0, a 32-token
prompt from seed 0, 16 greedy tokens through a paged KV cache of 16-position blocks."""
import numpy as np
import pytest

from poot_b200.models.config import tiny_llama
from poot_b200.models.model import Model, StepSpec
from poot_b200.oracle.runner import OracleSession, random_weights_f32


@pytest.fixture(scope="module")
def setup():
    model = Model(tiny_llama())
    weights = random_weights_f32(model, seed=0, std=0.02)
    prompt = np.random.default_rng(0).integers(0, 32000, size=32).astype(np.int32)
    return model, weights, prompt


def test_trace_validates_and_counts(setup):
    model, _, _ = setup
    g = model.trace(StepSpec(rows=1, tokens=4, capacity=64))
    g.validate()
    counts = g.summary()
    assert counts["matmul"] == 2 * (4 + 2 + 3) + 1      # q k v o + scores/pv + gate up down per layer, + head
    assert counts["scatter_update"] == 4 and counts["gather"] >= 7
    assert len(g.digest()) == 16


def test_greedy_generation_paged(setup):
    model, weights, prompt = setup
    s = OracleSession(model, weights, capacity=64, paged=True)
    out = s.generate(prompt, 16)
    assert len(out) == 16 and all(0 <= t < 32000 for t in out)
    # determinism: a second session reproduces the tokens
    assert OracleSession(model, weights, capacity=64, paged=True).generate(prompt, 16) == out


def test_decode_by_steps_equals_one_shot_prefill(setup):
    model, weights, prompt = setup
    one = OracleSession(model, weights, capacity=64).step(prompt[None, :])
    s = OracleSession(model, weights, capacity=64)
    s.step(prompt[None, :20])
    for t in range(20, 32):
        last = s.step(prompt[None, t:t + 1])
    np.testing.assert_allclose(last, one, rtol=1e-4, atol=2e-5)
    assert int(np.argmax(last)) == int(np.argmax(one))


def test_paged_equals_contiguous_bit_exact(setup):
    model, weights, prompt = setup
    order = [3, 0, 2, 1]          # a shuffled block table: movement must not change a single bit
    a = OracleSession(model, weights, capacity=64, paged=True, block_order=order).step(prompt[None, :])
    b = OracleSession(model, weights, capacity=64, paged=False).step(prompt[None, :])
    assert np.array_equal(a, b)


def test_narrow_precision_stays_close_to_exact(setup):
    from poot_b200.oracle.eval import EvalOptions
    model, weights, prompt = setup
    exact = OracleSession(model, weights, capacity=64).step(prompt[None, :])
    narrow = OracleSession(model, weights, capacity=64, options=EvalOptions(matmul_precision="narrow")).step(prompt[None, :])
    split = OracleSession(model, weights, capacity=64, options=EvalOptions(matmul_precision="split")).step(prompt[None, :])
    assert np.abs(narrow - exact).max() < 2e-2
    assert np.abs(split - exact).max() < np.abs(narrow - exact).max()
