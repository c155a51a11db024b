"""The compiled plan drives the engine: for the plain decoder families the step is a walk over the launch list lowered
from ``compile_graph``'s plans (``plan/lower.py`` -> ``runtime/program.py``), token-identical to the hand-sequenced
program, with the same launch count, over one arena laid out by lifetime colouring."""
import pytest
import torch

from poot_b200.models.config import DecoderConfig
from poot_b200.models.model import Model, StepSpec
from poot_b200.plan.compile import compile_graph
from poot_b200.plan.lower import lower
from poot_b200.runtime.engine import DecoderEngine, StepShape
from poot_b200.runtime.session import FixedBatchSession
from poot_b200.runtime.weights import random_weights
from poot_b200.utils.kernel_emulation import emulated_kernels

BASE = dict(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048, max_position=256)
FAMILIES = {
    "llama": {},
    "qwen2 (q/k/v bias, tied head)": dict(attn_bias=True, tie_embeddings=True),
    "qwen3 (per-head q/k norm)": dict(qk_norm=True),
    "mixtral (routed experts)": dict(n_experts=4, top_k=2, moe_ffn=128),
    "partial rotary": dict(rope_dim=32),
}


def _run(cfg, use_program: bool, batch=3, prompt=21, steps=3):
    w = random_weights(cfg, "cpu", seed=1, std=0.05)
    eng = DecoderEngine(w, num_blocks=32, max_seqs=4, max_tokens=160, max_blocks_per_seq=8, device="cpu", use_graphs=False)
    if not use_program:
        eng.program = None
    s = FixedBatchSession(eng, batch, 96)
    g = torch.Generator().manual_seed(2)
    prompts = torch.randint(0, cfg.vocab, (batch, prompt), generator=g, dtype=torch.int32)
    out = [s.prefill_fast(prompts).clone()]
    counts = [eng.launches_per_step[eng._key(StepShape(batch * prompt, batch))]]
    logits = [eng.logits_local[:batch].clone()]
    for _ in range(steps):
        out.append(s.decode(out[-1][:, 0].tolist()).clone())
        logits.append(eng.logits_local[:batch].clone())
    counts.append(eng.launches_per_step[eng._key(StepShape(batch, batch))])
    return torch.stack(out), torch.stack(logits), counts, eng


@pytest.mark.parametrize("name", list(FAMILIES))
def test_plan_walk_equals_the_hand_sequenced_program(name):
    cfg = DecoderConfig(**BASE, **FAMILIES[name])
    with emulated_kernels():
        got, got_logits, got_counts, eng = _run(cfg, True)
        want, want_logits, want_counts, _ = _run(cfg, False)
    assert eng.program is not None, "the family should run the compiled plan"
    assert torch.equal(got, want)
    assert torch.equal(got_logits, want_logits)          # bit-identical: the same launchers in the same order
    assert got_counts == want_counts


def test_launch_list_follows_the_plans_and_the_arena_is_coloured():
    cfg = DecoderConfig(**BASE)
    g = Model(cfg).trace(StepSpec(rows=2, tokens=2, capacity=64, paged=True, pool_slots=128))
    prog = compile_graph(g)
    lp = lower(prog)
    kinds = [l.op for l in lp.launches]
    per_layer = ["rmsnorm", "gemm", "rope_kv", "attention", "gemm", "rmsnorm", "gemm", "gemm"]
    assert kinds == ["embed"] + per_layer * cfg.n_layers + ["rows", "rmsnorm", "gemm"]
    # every dispatching equation of the plan is run by exactly one launch
    dispatching = {k for k, p in enumerate(prog.plans) if p.kind == "dispatch"}
    ran = [l.eqn for l in lp.launches if l.op != "rows"] + [c for l in lp.launches for c in l.covers]
    assert sorted(ran) == sorted(dispatching)
    # merged siblings name all their weights in row order; epilogues come from the plan
    qkv = lp.launches[2]
    assert qkv.weights == ("layers.0.attn_q", "layers.0.attn_k", "layers.0.attn_v") and qkv.width == (4 + 2 + 2) * 64
    assert [l.epi for l in lp.launches if l.op == "gemm"][:4] == ["store", "resid", "swiglu", "resid"]
    assert lp.launches[-1].epi == "f32" and lp.launches[-1].weights == ("lm_head",)
    # the residual stream is updated in place, and values with disjoint lifetimes share bytes
    o_proj = lp.launches[5]
    assert lp.row_bytes[o_proj.out] == lp.row_bytes[o_proj.resid]
    assert lp.arena_row_bytes < lp.sum_row_bytes / 2
    with emulated_kernels():
        w = random_weights(cfg, "cpu", seed=1, std=0.05)
        eng = DecoderEngine(w, num_blocks=32, max_seqs=4, max_tokens=160, max_blocks_per_seq=8, device="cpu", use_graphs=False)
    assert eng.program.arena_bytes < eng.program.separate_bytes / 2


def test_families_outside_the_lowering_keep_the_hand_sequenced_program():
    with emulated_kernels():
        for extra in (dict(block="post"), dict(attn_softcap=30.0, final_softcap=20.0), dict(act="gelu_tanh")):
            cfg = DecoderConfig(**BASE, **extra)
            w = random_weights(cfg, "cpu", seed=1, std=0.05)
            eng = DecoderEngine(w, num_blocks=8, max_seqs=2, max_tokens=64, max_blocks_per_seq=4, device="cpu", use_graphs=False)
            assert eng.program is None
