"""Planner passes that decide numerics and limits, each checked against the CPU oracle (bit-identical results):
operand precision, narrow storage, range witnesses, legalization."""
import numpy as np
import pytest

from poot_b200.models.config import DecoderConfig
from poot_b200.models.model import Model, StepSpec
from poot_b200.oracle.eval import EvalOptions, eval_graph
from poot_b200.oracle.runner import random_weights_f32
from poot_b200.plan import compile_graph
from poot_b200.plan.numerics import (LegalizeRefused, Limits, bind_legalized, check_narrow_ranges, failed_witnesses, legalize,
                                     select_operand_precision, store_narrowed_activations)


def _cfg(**kw):
    base = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=128, vocab=256, max_position=64)
    base.update(kw)
    return DecoderConfig(**base)


def _inputs(model, g, tokens=5, seed=0):
    rng = np.random.default_rng(seed)
    w = random_weights_f32(model, seed=1, std=0.2)
    ins = dict(w)
    T = tokens
    for i in g.inputs:
        if i.storage == "slot":
            shape = g.types[i.value].shape
            if i.slot == "token":
                ins[i.name] = rng.integers(0, model.cfg.vocab, shape)
            elif i.slot == "pos":
                ins[i.name] = np.arange(T).reshape(shape)
            else:
                ins[i.name] = np.arange(int(np.prod(shape))).reshape(shape) % max(1, g.types[i.value].shape[-1])
        elif i.storage == "state":
            ins[i.name] = np.zeros(g.types[i.value].shape, np.float32)
    return ins


def _graph(cfg, tokens=5):
    model = Model(cfg)
    g = model.trace(StepSpec(rows=1, tokens=tokens, capacity=16))
    return model, g


def test_precision_policy_is_a_permission_and_router_pins_stay_exact():
    model, g = _graph(_cfg(n_experts=4, top_k=2, moe_ffn=32))
    p = compile_graph(g).graph
    counts = select_operand_precision(p, "narrow")
    assert counts["pinned"] == model.cfg.n_layers            # the routers' logits stay exact under any policy
    assert counts["narrow"] > 0 and counts["exact"] == 0
    q = compile_graph(g).graph
    c2 = select_operand_precision(q, "exact")
    assert c2["exact"] == counts["narrow"] and c2.get("narrow", 0) == 0
    # the oracle follows the attribute: exact policy == the exact lane
    ins = _inputs(model, q)
    a = eval_graph(q, ins).outputs["logits"]
    b = eval_graph(compile_graph(g).graph, ins, EvalOptions(matmul_precision="exact")).outputs["logits"]
    assert np.array_equal(a, b)
    with pytest.raises(ValueError):
        select_operand_precision(q, "fp4")


def test_values_every_reader_narrows_are_stored_narrow_and_nothing_changes():
    model, g = _graph(_cfg())
    p = compile_graph(g).graph
    select_operand_precision(p, "narrow")
    ins = _inputs(model, p)
    before = eval_graph(p, ins).outputs["logits"]
    n = store_narrowed_activations(p)
    assert n >= 2 * model.cfg.n_layers                        # at least every norm output and every gated activation
    stored = [e for e in p.eqns if e.attrs.get("store") == "bf16"]
    assert any(e.op == "fused_row" for e in stored) and any(e.op in ("fused", "dense_contraction") for e in stored)
    assert not any(e.attrs.get("store") for e in p.eqns if e.outputs[0] in {o.value for o in p.outputs})   # logits stay f32
    assert np.array_equal(eval_graph(p, ins).outputs["logits"], before)
    q = compile_graph(g).graph
    select_operand_precision(q, "exact")
    assert store_narrowed_activations(q) == 0                # under an exact policy no reader narrows


def test_range_witnesses_name_the_operand_that_left_the_range():
    model, g = _graph(_cfg())
    p = compile_graph(g).graph
    select_operand_precision(p, "narrow")
    ins = _inputs(model, p)
    ref = eval_graph(p, ins).outputs["logits"]
    names = check_narrow_ranges(p)
    p.validate()
    assert names and all(n.startswith("narrow_range.") for n in names)
    out = eval_graph(p, ins).outputs
    assert np.array_equal(out["logits"], ref) and failed_witnesses(out) == []
    bad = dict(ins)
    bad["layers.1.ffn_norm"] = np.full_like(ins["layers.1.ffn_norm"], np.inf)      # the second layer's FFN input overflows
    fired = failed_witnesses(eval_graph(p, bad).outputs)
    assert fired and any(".l1." in n for n in fired) and not any(".l0." in n for n in fired)


def test_oversized_weights_are_split_into_row_chunks_and_the_rest_is_refused():
    model, g = _graph(_cfg())
    p = compile_graph(g).graph
    ins = _inputs(model, p)
    ref = eval_graph(p, ins).outputs["logits"]
    head_bytes = model.cfg.vocab * model.cfg.hidden * 4
    split = legalize(p, Limits(max_buffer_bytes=head_bytes // 3))
    p.validate()
    assert split == {"lm_head": 4} or split.get("lm_head", 0) >= 3
    assert not any(i.name == "lm_head" for i in p.inputs)       # the program's inputs are the chunks now
    out = eval_graph(p, bind_legalized(ins, p)).outputs["logits"]
    # each output column is the same dot product as before; only the host BLAS blocks a narrower matrix differently
    assert np.allclose(out, ref, rtol=1e-6, atol=1e-6)
    assert legalize(compile_graph(g).graph) == {}               # nothing of this model exceeds a B200's limits
    with pytest.raises(LegalizeRefused):
        legalize(compile_graph(g).graph, Limits(max_buffer_bytes=16))


def test_compile_options_run_the_numerics_passes():
    from poot_b200.plan import CompileOptions
    model, g = _graph(_cfg())
    prog = compile_graph(g, CompileOptions(precision="narrow", check_ranges=True, limits=Limits(max_buffer_bytes=20000)))
    assert prog.log["select_operand_precision"]["narrow"] > 0 and prog.log["store_narrowed_activations"] > 0
    assert prog.log["check_narrow_ranges"] > 0 and prog.log["legalize"]
    assert any(o.role == "witness" for o in prog.graph.outputs)
    plain = compile_graph(g)
    assert "legalize" not in plain.log and not any(o.role == "witness" for o in plain.graph.outputs)
