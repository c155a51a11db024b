"""The engine's kernel program on the CPU: ``emulated_kernels`` swaps the device kernels' entry points for host
restatements with the same signatures and buffer layouts, so the unmodified engine (buffer binding, launch order,
epilogue choices, K/V paging through block tables, tile cutting for the prefill attention, chained decode, the
sampler suffix, the serving driver on top) is compared with the fp32 restatement of the model without a GPU.  The
kernels themselves are checked on the device (tests marked ``gpu``)."""
import numpy as np
import pytest
import torch

from poot_b200.models.config import DecoderConfig
from poot_b200.utils.kernel_emulation import emulated_kernels


def _cfg(**kw):
    base = dict(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512, max_position=256)
    base.update(kw)
    return DecoderConfig(**base)


def _engine(cfg, batch, max_len, max_tokens, seed=0):
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    w = random_weights(cfg, "cpu", seed=seed, std=0.05)
    bps = (max_len + 15) // 16
    eng = DecoderEngine(w, num_blocks=batch * bps + 1, max_seqs=batch, max_tokens=max_tokens, max_blocks_per_seq=bps,
                        device="cpu", use_graphs=False)
    return w, eng, FixedBatchSession(eng, batch, max_len)


VARIANTS = {
    "llama": {},
    "head-dim-128-flash-tiles": dict(n_heads=2, n_kv_heads=1, head_dim=128, hidden=256),
    "qk-norm-window": dict(qk_norm=True, sliding_window=8),
    "per-layer-windows": dict(layer_windows=[6, 0]),
    "scale-override-softcap": dict(attn_scale=0.2, attn_softcap=20.0),
    "qkv-bias-multipliers": dict(attn_bias=True, embed_scale=3.0, residual_scale=0.5, logit_scale=0.25),
    "partial-rotary": dict(rope_dim=32),
    "moe": dict(n_experts=4, top_k=2, moe_ffn=128),
    "moe-not-renormalised": dict(n_experts=4, top_k=2, moe_ffn=128, norm_topk_prob=False),
}


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_prefill_then_decode_matches_the_fp32_restatement(name):
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = _cfg(**VARIANTS[name])
    with emulated_kernels():
        w, eng, sess = _engine(cfg, batch=2, max_len=64, max_tokens=64)
        g = torch.Generator().manual_seed(0)
        prompts = torch.randint(0, cfg.vocab, (2, 21), generator=g, dtype=torch.int32)
        picked = sess.prefill_fast(prompts)
        for b in range(2):
            ref = forward_logits(w, prompts[b])[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), (name, "prefill", err)
            assert picked[b, 1] == -1
        nxt = torch.randint(0, cfg.vocab, (2, 3), generator=g, dtype=torch.int32)
        for t in range(3):
            sess.decode(nxt[:, t].tolist())
        for b in range(2):
            ref = forward_logits(w, torch.cat([prompts[b], nxt[b]]))[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), (name, "decode", err)


def test_chained_decode_equals_stepwise_decode():
    cfg = _cfg()
    with emulated_kernels():
        g = torch.Generator().manual_seed(3)
        prompts = torch.randint(0, cfg.vocab, (2, 9), generator=g, dtype=torch.int32)
        _, eng_a, a = _engine(cfg, 2, 64, 32)
        first = a.prefill_fast(prompts)[:, 0].tolist()
        toks, cur = [], first
        for _ in range(5):
            cur = a.decode(cur)[:, 0].tolist()
            toks.append(cur)
        _, eng_b, b = _engine(cfg, 2, 64, 32)
        first_b = b.prefill_fast(prompts)[:, 0].tolist()
        assert first_b == first
        chained = b.decode_chain(first_b, 5)
        assert [list(map(int, chained[i])) for i in range(5)] == toks if chained is not None else True
        assert eng_b.picked[:2, 0].tolist() == toks[-1]


def test_device_gaps_are_refused_by_the_engine():
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import UnsupportedOnDevice, random_weights
    cfg = _cfg(attn_sinks=True)
    with emulated_kernels():
        w = random_weights(_cfg(), "cpu", seed=0)
        w.cfg = cfg
        with pytest.raises(UnsupportedOnDevice) as e:
            DecoderEngine(w, 8, 1, 16, 4, device="cpu", use_graphs=False)
    assert "sinks" in str(e.value)


def test_serving_driver_over_the_emulated_engine_matches_greedy_reference():
    """Driver -> DeviceStepEngine -> engine: chunked prefill of two sequences sharing steps, then decode."""
    from poot_b200.driver.driver import Driver
    from poot_b200.driver.engines import DeviceStepEngine
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.oracle.torch_ref import forward_logits
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import random_weights
    cfg = _cfg()
    with emulated_kernels():
        w = random_weights(cfg, "cpu", seed=1, std=0.05)
        eng = DecoderEngine(w, num_blocks=16, max_seqs=2, max_tokens=16 + 2, max_blocks_per_seq=4, device="cpu", use_graphs=False)
        step_engine = DeviceStepEngine(eng)
        drv = Driver(step_engine, 16, 2, 64, cfg.vocab, prefill_chunk=16, eos_token=None)
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (37, 6)]
        sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
        ids = [drv.open(p, sp) for p in prompts]
        got = {i: [] for i in ids}
        live = set(ids)
        while live:
            for r in drv.step(sorted(live)):
                if r.token is None:
                    continue
                drv.commit(r.seq_id, [r.token])
                got[r.seq_id].append(r.token)
                if drv.finished(r.seq_id, r.token):
                    drv.release(r.seq_id)
                    live.discard(r.seq_id)
    for i, p in zip(ids, prompts):
        seq = list(p)
        for t in got[i]:
            ref = forward_logits(w, torch.tensor(seq, dtype=torch.int32))[-1]
            top2 = torch.topk(ref, 2).values
            if float(top2[0] - top2[1]) > 0.05:        # bf16 storage can flip a near-tie
                assert t == int(ref.argmax())
            seq.append(t)


@pytest.mark.parametrize("kw", [{}, dict(n_experts=4, top_k=2, moe_ffn=128)], ids=["dense", "moe"])
def test_long_prefill_takes_the_tiled_split_k_route(kw):
    """More than 128 tokens in a step: the tiled GEMM, split-K partial slices folded into the next norm, expert
    chunks of 128 rows."""
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = _cfg(hidden=1024, ffn=512, n_heads=4, n_kv_heads=2, head_dim=64, **kw)
    with emulated_kernels():
        w, eng, sess = _engine(cfg, batch=2, max_len=96, max_tokens=192)
        g = torch.Generator().manual_seed(4)
        prompts = torch.randint(0, cfg.vocab, (2, 80), generator=g, dtype=torch.int32)
        sess.prefill_fast(prompts)
        for b in range(2):
            ref = forward_logits(w, prompts[b])[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), err


HF_BASE = {"hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
           "intermediate_size": 384, "vocab_size": 512, "rms_norm_eps": 1e-5, "max_position_embeddings": 128}
HF_FAMILIES = {
    "gemma2": {"model_type": "gemma2", "query_pre_attn_scalar": 48, "sliding_window": 8, "attn_logit_softcapping": 1.0,
               "final_logit_softcapping": 10.0},
    "gemma3": {"model_type": "gemma3_text", "query_pre_attn_scalar": 48, "sliding_window": 8, "num_hidden_layers": 3,
               "layer_types": ["sliding_attention", "sliding_attention", "full_attention"], "rope_local_base_freq": 10000.0,
               "rope_theta": 1000000.0},
    "olmo2": {"model_type": "olmo2"},
    "olmoe": {"model_type": "olmoe", "num_experts": 4, "num_experts_per_tok": 2, "intermediate_size": 128},
    "smollm3-nope-layer": {"model_type": "smollm3", "no_rope_layers": [1, 0]},
    "minimax_m2": {"model_type": "minimax_m2", "num_local_experts": 4, "num_experts_per_tok": 2, "intermediate_size": 128},
    "granite": {"model_type": "granite", "embedding_multiplier": 6.0, "residual_multiplier": 0.5, "logits_scaling": 4.0,
                "attention_multiplier": 0.1},
}


@pytest.mark.parametrize("name", sorted(HF_FAMILIES))
def test_family_blocks_on_the_engine_match_the_graph_oracle(name):
    """Families beyond the plain pre-norm SwiGLU layer (sandwich and post norms, GeGLU, soft caps, two rope bases,
    projection-wide q/k norms, layers without rope): the engine's program against the graph oracle, which is itself
    checked against the Hugging Face implementations."""
    from poot_b200.models.model import StepSpec
    from poot_b200.models.registry import Registry
    from poot_b200.oracle.runner import OracleSession, random_weights_f32
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import from_named_tensors
    model = Registry.builtin().resolve_hf({**HF_BASE, **HF_FAMILIES[name]})
    cfg = model.cfg
    assert cfg.device_gaps() == [], cfg.device_gaps()
    w = random_weights_f32(model, seed=2, std=0.08)
    for k in w:
        if k.endswith("select_bias"):
            w[k] = (0.3 * np.random.default_rng(1).standard_normal(w[k].shape)).astype(np.float32)
        if k.endswith("norm"):
            w[k] = (1.0 + 0.1 * np.random.default_rng(len(k)).standard_normal(w[k].shape)).astype(np.float32)
    w = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}     # what the device will hold
    named = {k: torch.from_numpy(v) for k, v in w.items()}
    for l in range(cfg.n_layers if cfg.is_moe else 0):
        p = f"layers.{l}."
        for e in range(cfg.n_experts):
            named[p + f"experts.{e}.gate"] = named[p + "experts_in"][e, :cfg.moe_ffn]
            named[p + f"experts.{e}.up"] = named[p + "experts_in"][e, cfg.moe_ffn:]
            named[p + f"experts.{e}.down"] = named[p + "experts_out"][e]
    toks = np.random.default_rng(7).integers(0, cfg.vocab, (1, 23))
    sess = OracleSession(model, w, capacity=32)
    ref = torch.from_numpy(sess.step(toks))[0]
    with emulated_kernels():
        dw = from_named_tensors(cfg, named, "cpu")
        eng = DecoderEngine(dw, num_blocks=4, max_seqs=1, max_tokens=32, max_blocks_per_seq=2, device="cpu", use_graphs=False)
        s = FixedBatchSession(eng, 1, 32)
        s.prefill_fast(torch.from_numpy(toks[:, :20]).int())
        for t in range(20, 23):
            s.decode([int(toks[0, t])])
        got = eng.logits[0]
    err = (got - ref).abs().max().item()
    assert err < 0.02 * max(1.0, ref.abs().max().item()), (name, err, ref.abs().max().item())


def test_pipeline_stages_reproduce_the_single_device_run():
    """Three pipeline stages (one thread each, queues as links) over the emulated kernels: the first stage embeds and
    gets the sampled tokens back, the middle stage only transforms the residual stream, the last stage samples; the
    logits and tokens equal the unsplit engine's, for a prefill step and decode steps through each stage's own K/V."""
    import threading
    from poot_b200.driver.placement import Placement, pipeline_cuts
    from poot_b200.parallel.pipeline import LocalLink
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import StageSpec, random_weights
    cfg = _cfg(n_layers=5, layer_windows=[0, 6, 0, 6, 0])
    cuts = pipeline_cuts(cfg, 3)
    assert [b - a for a, b in cuts] in ([1, 2, 2], [2, 2, 1], [2, 1, 2]) and cuts[0][0] == 0 and cuts[-1][1] == 5
    Placement.parse("pipeline:0,1,2").validate(cfg)
    g = torch.Generator().manual_seed(11)
    prompts = torch.randint(0, cfg.vocab, (2, 18), generator=g, dtype=torch.int32)
    nxt = torch.randint(0, cfg.vocab, (2, 2), generator=g, dtype=torch.int32)

    def drive(sess):
        out = [sess.prefill_fast(prompts).clone()]
        for t in range(2):
            out.append(sess.decode(nxt[:, t].tolist()).clone())
        return out

    with emulated_kernels():
        _, whole, s = _engine(cfg, 2, 64, 48)
        want = drive(s)
        want_logits = whole.logits[:2].clone()
        queues, engines, results = {}, [], {}
        for i, (l0, l1) in enumerate(cuts):
            st = StageSpec(i, 3, l0, l1)
            w = random_weights(cfg, "cpu", seed=0, std=0.05, stage=st)
            assert len(w.layers) == l1 - l0 and (w.embed is not None) == st.first and (w.lm_head is not None) == st.last
            engines.append(DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=48, max_blocks_per_seq=4, device="cpu",
                                         use_graphs=False, link=LocalLink(queues, i, 3)))

        def stage(i):
            results[i] = drive(FixedBatchSession(engines[i], 2, 64))
        threads = [threading.Thread(target=stage, args=(i,)) for i in range(3)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=120)
        assert sorted(results) == [0, 1, 2]
    for a, b in zip(results[0], want):            # the driver's stage holds the tokens the last stage sampled
        assert torch.equal(a, b)
    assert torch.equal(engines[2].logits[:2], want_logits)
    assert engines[0].kv.buf.shape[0] == cuts[0][1] - cuts[0][0] and engines[0].link.sent_bytes > 0


def test_bench_driver_path_runs_on_the_emulated_engine():
    """The benchmark's end-to-end arm (Driver.open / step / commit over DeviceStepEngine) on a tiny model: chunked
    prefill of the whole batch, warm-up, timed steps, release."""
    import importlib.util
    import os
    import time
    spec = importlib.util.spec_from_file_location("poot_bench", os.path.join(os.path.dirname(__file__), "..", "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cfg = _cfg()
    calls = []

    def timed(fn, n):
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        calls.append(n)
        return (time.perf_counter() - t0) * 1e3

    with emulated_kernels():
        B, P = 3, 40
        max_len = P + 64
        bps = (max_len + 15) // 16
        from poot_b200.runtime.engine import DecoderEngine
        from poot_b200.runtime.weights import random_weights
        w = random_weights(cfg, "cpu", seed=0, std=0.05)
        eng = DecoderEngine(w, num_blocks=B * bps + bps, max_seqs=B, max_tokens=512 + B, max_blocks_per_seq=bps, device="cpu",
                            use_graphs=False)
        prompts = torch.randint(0, cfg.vocab, (B, P), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
        r = bench.driver_e2e(eng, cfg, B, prompts, 2, 3, max_len, timed)
    assert calls == [3] and r["tok_s"] > 0 and r["ms_per_step"] > 0
