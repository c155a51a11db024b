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
    "head-dim-256-general-attention": dict(n_heads=2, n_kv_heads=1, head_dim=256, hidden=256, sliding_window=12, attn_softcap=30.0),
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
    cfg = _cfg(mlp_bias=True)
    with emulated_kernels():
        w = random_weights(_cfg(), "cpu", seed=0)
        w.cfg = cfg
        with pytest.raises(UnsupportedOnDevice) as e:
            DecoderEngine(w, 8, 1, 16, 4, device="cpu", use_graphs=False)
    assert "biases of a gated dense FFN" in str(e.value)


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
    "qwen3_5": {"model_type": "qwen3_5_text", "num_hidden_layers": 4, "layer_types": ["linear_attention", "full_attention"] * 2,
                "linear_num_value_heads": 4, "linear_num_key_heads": 2, "linear_key_head_dim": 64, "linear_value_head_dim": 64,
                "linear_conv_kernel_dim": 4, "rope_parameters": {"rope_theta": 10000.0, "partial_rotary_factor": 0.5, "rope_type": "default"}},
    "qwen3next": {"model_type": "qwen3_next", "num_hidden_layers": 2, "layer_types": ["linear_attention", "full_attention"],
                  "linear_num_value_heads": 4, "linear_num_key_heads": 2, "linear_key_head_dim": 64, "linear_value_head_dim": 64,
                  "num_experts": 16, "num_experts_per_tok": 10, "moe_intermediate_size": 64, "shared_expert_intermediate_size": 128,
                  "partial_rotary_factor": 0.25},
    "deepseek2": {"model_type": "deepseek_v2", "n_routed_experts": 8, "num_experts_per_tok": 3, "moe_intermediate_size": 64,
                  "first_k_dense_replace": 1, "kv_lora_rank": 64, "q_lora_rank": None, "qk_rope_head_dim": 32,
                  "qk_nope_head_dim": 64, "v_head_dim": 64, "n_shared_experts": 2, "num_key_value_heads": 4},
    "deepseek3": {"model_type": "deepseek_v3", "n_routed_experts": 8, "num_experts_per_tok": 3, "moe_intermediate_size": 64,
                  "first_k_dense_replace": 1, "kv_lora_rank": 64, "q_lora_rank": 96, "qk_rope_head_dim": 32, "qk_nope_head_dim": 64,
                  "v_head_dim": 64, "n_shared_experts": 1, "n_group": 4, "topk_group": 2, "num_key_value_heads": 4},
    "gpt_oss": {"model_type": "gpt_oss", "num_local_experts": 8, "num_experts_per_tok": 2, "intermediate_size": 128, "sliding_window": 6,
                "layer_types": ["sliding_attention", "full_attention"], "attention_bias": True,
                "rope_parameters": {"rope_type": "yarn", "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False,
                                    "original_max_position_embeddings": 32, "rope_theta": 10000.0}},
    "mpt": {"model_type": "mpt", "d_model": 256, "n_heads": 4, "n_layers": 2, "vocab_size": 512, "max_seq_len": 128,
            "attn_config": {"alibi": True}},
    "bloom": {"model_type": "bloom", "hidden_size": 384, "n_head": 6, "n_layer": 2, "vocab_size": 512},
    "nemotron_h": {"model_type": "nemotron_h", "hybrid_override_pattern": "M-*E", "mamba_num_heads": 4, "mamba_head_dim": 32,
                   "ssm_state_size": 16, "n_groups": 2, "conv_kernel": 4, "n_routed_experts": 4, "num_experts_per_tok": 2,
                   "moe_intermediate_size": 64, "moe_shared_expert_intermediate_size": 96, "layer_norm_epsilon": 1e-5},
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
    model = Registry.builtin().resolve_hf(HF_FAMILIES[name] if name in ("mpt", "bloom") else {**HF_BASE, **HF_FAMILIES[name]})
    cfg = model.cfg
    assert cfg.device_gaps() == [], cfg.device_gaps()
    w = random_weights_f32(model, seed=2, std=0.08)
    for k in w:
        if k.endswith("select_bias"):
            w[k] = (0.3 * np.random.default_rng(1).standard_normal(w[k].shape)).astype(np.float32)
        if k.endswith(("norm", "norm_w")):
            w[k] = (1.0 + 0.1 * np.random.default_rng(len(k)).standard_normal(w[k].shape)).astype(np.float32)
        if k.endswith(("gdn_a_log", "ssm_a_log")):
            w[k] = np.log(np.random.default_rng(3).uniform(0.5, 4.0, w[k].shape)).astype(np.float32)
    w = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}     # what the device will hold
    named = {k: torch.from_numpy(v) for k, v in w.items()}
    for l in [l for l in range(cfg.n_layers) if cfg.has_ffn(l) and cfg.moe_layer(l)]:
        p = f"layers.{l}."
        for e in range(cfg.n_experts):
            named[p + f"experts.{e}.gate"] = named[p + "experts_in"][e, :cfg.moe_ffn]
            named[p + f"experts.{e}.up"] = named[p + "experts_in"][e, cfg.moe_ffn:] if cfg.gated_ffn else named[p + "experts_in"][e]
            named[p + f"experts.{e}.down"] = named[p + "experts_out"][e]
    # routed experts make the model discontinuous: where two router scores nearly tie, bf16 rounding can pick the other
    # expert and move the logits by several percent; the token seed of such a family avoids a near-tie on its last steps
    toks = np.random.default_rng({"gpt_oss": 9}.get(name, 7)).integers(0, cfg.vocab, (1, 23))
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


def make_adapter(cfg, rng, name, r, roles):
    from poot_b200.load.lora import LoraAdapter
    d = {}
    for l in range(cfg.n_layers):
        for role, (o, i) in roles.items():
            d[f"layers.{l}.{role}"] = ((rng.standard_normal((r, i)) * 0.2).astype(np.float32),
                                        (rng.standard_normal((o, r)) * 0.2).astype(np.float32))
    return LoraAdapter(name, r, 0.5, d)


def adapter_roles(cfg):
    H, F = cfg.hidden, cfg.ffn
    return {"attn_q": (cfg.q_size, H), "attn_k": (cfg.kv_size, H), "attn_v": (cfg.kv_size, H), "attn_o": (H, cfg.q_size),
            "ffn_gate": (F, H), "ffn_up": (F, H), "ffn_down": (H, F)}


def merged_weights(cfg, w, ad):
    """Reference: the engine's fused layouts with the adapter's delta merged in."""
    import copy
    m = copy.deepcopy(w)
    q, kv = cfg.q_size, cfg.kv_size
    for l, L in enumerate(m.layers):
        p = f"layers.{l}."
        dl = lambda role: torch.from_numpy(ad.delta(p + role)).to(L.wo.device) if (p + role) in ad.deltas else None
        wqkv = L.wqkv.float()
        for role, (a, b) in (("attn_q", (0, q)), ("attn_k", (q, q + kv)), ("attn_v", (q + kv, q + 2 * kv))):
            if dl(role) is not None:
                wqkv[a:b] += dl(role)
        L.wqkv = wqkv.to(torch.bfloat16)
        if dl("attn_o") is not None:
            L.wo = (L.wo.float() + dl("attn_o")).to(torch.bfloat16)
        wgu = L.wgu.float()
        if dl("ffn_gate") is not None:
            wgu[0::2] += dl("ffn_gate")
        if dl("ffn_up") is not None:
            wgu[1::2] += dl("ffn_up")
        L.wgu = wgu.to(torch.bfloat16)
        if dl("ffn_down") is not None:
            L.wdown = (L.wdown.float() + dl("ffn_down")).to(torch.bfloat16)
    return m


def test_rows_of_one_step_use_different_resident_adapters():
    """Two sequences in the same steps, one per adapter, a third without any: each row's logits equal the model whose
    projections carry that adapter's merged delta (prefill and decode through the bank's grouped contractions)."""
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = _cfg()
    rng = np.random.default_rng(0)
    every = adapter_roles(cfg)
    ad_a = make_adapter(cfg, rng, "a", 8, every)
    ad_b = make_adapter(cfg, rng, "b", 4, {"attn_q": every["attn_q"], "attn_v": every["attn_v"], "ffn_down": every["ffn_down"]})
    merged = lambda w_, ad: merged_weights(cfg, w_, ad)

    with emulated_kernels():
        w, eng, sess = _engine(cfg, batch=3, max_len=64, max_tokens=96)
        bank = eng.enable_adapters(slots=4, max_rank=8)
        sa, sb = bank.load(ad_a), bank.load(ad_b)
        assert (sa, sb) == (0, 1) and bank.slot_of("b") == 1
        g = torch.Generator().manual_seed(0)
        prompts = torch.randint(0, cfg.vocab, (3, 17), generator=g, dtype=torch.int32)
        slots = [sa, sb, -1]
        T = 3 * 17
        assert bank.bind_rows(np.repeat(np.array(slots, np.int32), 17), T)
        from poot_b200.runtime.engine import StepShape
        # prefill with adapters: the session binds the inputs, the step shape carries the adapter flag
        B, L = prompts.shape
        pos = torch.arange(L, dtype=torch.int32).repeat(B)
        seq = torch.arange(B, dtype=torch.int32).repeat_interleave(L)
        sess.h_tokens[:T] = prompts.reshape(-1)
        sess.h_pos[:T], sess.h_seq[:T] = pos, seq
        blk = sess.block_tables_host[seq.long(), (pos // 16).long()]
        sess.h_slots[:T] = blk * 16 + pos % 16
        sess.h_ctx[:T] = pos + 1
        sess.h_lidx[:B] = torch.arange(B, dtype=torch.int64) * L + (L - 1)
        sess.lengths = [L] * B
        sess._step(StepShape(T, B, 0, lora=True))
        refs = [merged(w, ad_a), merged(w, ad_b), w]
        for b in range(3):
            ref = forward_logits(refs[b], prompts[b])[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), ("prefill", b, err)
        # the adapter matters: row 0 differs from the base model by more than the tolerance
        base = forward_logits(w, prompts[0])[-1]
        assert (eng.logits[0] - base).abs().max().item() > 0.1 * base.abs().max().item()
        # one decode step, one row per sequence
        nxt = torch.randint(0, cfg.vocab, (3,), generator=g, dtype=torch.int32)
        bank.bind_rows(np.array(slots, np.int32), 3)
        sess._bind_decode_inputs(nxt.tolist())
        sess.len_t = sess.len_t + 1
        sess._step(StepShape(3, 3, 0, lora=True))
        for b in range(3):
            ref = forward_logits(refs[b], torch.cat([prompts[b], nxt[b:b + 1]]))[-1]
            err = (eng.logits[b] - ref).abs().max().item()
            assert err < 0.03 * max(1.0, ref.abs().max().item()), ("decode", b, err)
        bank.unload("a")
        assert bank.names[:2] == [None, "b"]


def test_server_loads_adapters_and_requests_select_them_by_model_name(tmp_path):
    """HTTP server over the emulated engine: ``POST /v1/lora_adapters`` makes a PEFT directory resident, a request whose
    ``model`` names it decodes with it (and differs from the base model's answer), the adapter shows up under
    ``/v1/models``, cannot be deleted twice, and a sequence opened under it does not share prefix-cache blocks with the
    base model."""
    import json
    import urllib.request
    from poot_b200.driver.driver import Driver
    from poot_b200.driver.engines import DeviceStepEngine
    from poot_b200.load import safetensors as st
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import random_weights
    from poot_b200.serve.config import ServeConfig
    from poot_b200.serve.http import Server, ServerState
    from poot_b200.serve.metrics import Metrics
    from poot_b200.serve.scheduler import ServeEngine
    from poot_b200.tensor import DType
    from poot_b200.text.codec import ByteTokenizer
    cfg = _cfg(vocab=300)
    rng = np.random.default_rng(0)
    d = tmp_path / "adapter"
    d.mkdir()
    (d / "adapter_config.json").write_text(json.dumps({"peft_type": "LORA", "r": 4, "lora_alpha": 16}))
    tensors = {}
    for l in range(cfg.n_layers):
        for mod, (o, i) in (("self_attn.q_proj", (cfg.q_size, cfg.hidden)), ("mlp.down_proj", (cfg.hidden, cfg.ffn))):
            tensors[f"base_model.model.model.layers.{l}.{mod}.lora_A.weight"] = (DType.F32, (rng.standard_normal((4, i)) * 0.3).astype(np.float32))
            tensors[f"base_model.model.model.layers.{l}.{mod}.lora_B.weight"] = (DType.F32, (rng.standard_normal((o, 4)) * 0.3).astype(np.float32))
    st.write_safetensors(str(d / "adapter_model.safetensors"), tensors)
    key = tmp_path / "key"
    key.write_text("sesame")
    with emulated_kernels():
        w = random_weights(cfg, "cpu", seed=1, std=0.05)
        eng = DecoderEngine(w, num_blocks=24, max_seqs=2, max_tokens=34, max_blocks_per_seq=8, device="cpu", use_graphs=False)
        eng.enable_adapters(slots=2, max_rank=8)
        tk = ByteTokenizer(cfg.vocab)
        drv = Driver(DeviceStepEngine(eng), 24, 2, 128, cfg.vocab, prefill_chunk=32, eos_token=tk.eos)
        serve = ServeEngine(drv, tk, Metrics())
        scfg = ServeConfig(model="tiny", addr="127.0.0.1:0", lora_admin_key_file=str(key))
        server = Server(ServerState(serve, scfg, "tiny"))
        serve.start()
        server.start()
        try:
            def call(method, path, body=None, admin=False):
                req = urllib.request.Request(f"http://127.0.0.1:{server.port}{path}", None if body is None else json.dumps(body).encode(),
                                             {"Content-Type": "application/json", **({"Authorization": "Bearer sesame"} if admin else {})},
                                             method=method)
                try:
                    with urllib.request.urlopen(req, timeout=60) as r:
                        return r.status, json.loads(r.read())
                except urllib.error.HTTPError as e:
                    return e.code, json.loads(e.read())
            st_, _ = call("POST", "/v1/lora_adapters", {"name": "tuned", "path": str(d)})
            assert st_ in (401, 403)                                   # admin key required
            st_, body = call("POST", "/v1/lora_adapters", {"name": "tuned", "path": str(d)}, admin=True)
            assert st_ == 200 and body["slot"] == 0 and body["rank"] == 4, body
            st_, body = call("POST", "/v1/lora_adapters", {"name": "tuned", "path": str(d)}, admin=True)
            assert st_ == 409
            st_, models = call("GET", "/v1/models")
            assert [m["id"] for m in models["data"]] == ["tiny", "tuned"]
            ask = {"prompt": "the quick brown fox jumps", "max_tokens": 6, "temperature": 0, "ignore_eos": True}
            st_, base = call("POST", "/v1/completions", {**ask, "model": "tiny"})
            st_, tuned = call("POST", "/v1/completions", {**ask, "model": "tuned"})
            st_, base2 = call("POST", "/v1/completions", ask)
            assert st_ == 200 and base["choices"][0]["text"] == base2["choices"][0]["text"]
            assert tuned["choices"][0]["text"] != base["choices"][0]["text"]
            assert base2["usage"].get("prompt_tokens_details", {}).get("cached_tokens", 0) >= 16     # same identity: shared prefix
            assert tuned["usage"].get("prompt_tokens_details", {}).get("cached_tokens", 0) == 0      # other identity: none
            st_, _ = call("POST", "/v1/completions", {**ask, "model": "nobody"})
            assert st_ == 404
            st_, _ = call("DELETE", "/v1/lora_adapters/tuned", admin=True)
            assert st_ == 200
            st_, _ = call("DELETE", "/v1/lora_adapters/tuned", admin=True)
            assert st_ == 404
            st_, _ = call("POST", "/v1/completions", {**ask, "model": "tuned"})
            assert st_ == 404
        finally:
            server.shutdown()
            serve.drain(5)


@pytest.mark.parametrize("kw", [{}, dict(n_experts=4, top_k=2, moe_ffn=128)], ids=["dense", "moe"])
def test_planner_launch_census_equals_the_engine_launch_count(kw):
    """The planner's dispatch count for a decode step equals what the engine launches for it (the engine adds the
    two-stage greedy pick, which the traced graph exports logits for instead)."""
    from poot_b200.models.model import Model, StepSpec
    from poot_b200.plan import compile_graph
    from poot_b200.runtime.engine import StepShape
    cfg = _cfg(**kw)
    prog = compile_graph(Model(cfg).trace(StepSpec(rows=2, tokens=1, capacity=64)))
    with emulated_kernels():
        _, eng, sess = _engine(cfg, 2, 64, 32)
        sess.prefill_fast(torch.randint(0, cfg.vocab, (2, 9), generator=torch.Generator().manual_seed(0), dtype=torch.int32))
        sess.decode([1, 2])
        launched = eng.launches_per_step[eng._key(StepShape(2, 2, 0))]
    assert launched - 2 == prog.dispatches, (launched, prog.census)


def test_planner_census_of_the_row_grouped_expert_regime():
    """More (token, slot) rows than experts: routing, align and gather, two grouped GEMMs, scatter-combine."""
    from poot_b200.models.model import Model, StepSpec
    from poot_b200.plan import compile_graph
    from poot_b200.runtime.engine import StepShape
    cfg = _cfg(n_experts=4, top_k=2, moe_ffn=128)
    prog = compile_graph(Model(cfg).trace(StepSpec(rows=1, tokens=18, capacity=64, paged=True, pool_slots=128)))
    L = cfg.n_layers
    moe = {k: v for k, v in prog.census.items() if "moe" in k or "grouped" in k}
    assert moe == {"poot_moe_route": L, "poot_moe_align": L, "poot_moe_gather_rows": L, "poot_gemm_skinny_grouped": 2 * L,
                   "poot_moe_scatter_combine": L}
    counts = {}
    with emulated_kernels():
        for name, c in (("moe", cfg), ("dense", _cfg())):
            _, eng, sess = _engine(c, 2, 64, 48)
            sess.prefill_fast(torch.randint(0, c.vocab, (2, 9), generator=torch.Generator().manual_seed(0), dtype=torch.int32))
            counts[name] = eng.launches_per_step[eng._key(StepShape(18, 2, 0))]
    # a routed block is the router GEMM + six launches where the dense FFN has two
    assert counts["moe"] - counts["dense"] == L * (7 - 2), counts


def test_encoder_engine_matches_the_graph_oracle(tmp_path):
    """BERT on the device engine's kernels (restated on the host): ragged batch, K/V of each sequence in its own pool
    blocks, every token seeing its whole sequence; hidden states, pooled embeddings and a cross-encoder's scores against
    the graph oracle, which is itself checked against the Hugging Face model."""
    from poot_b200.embed import Embedder, PairTokenizer
    from poot_b200.models.encoder import EncoderConfig, EncoderModel
    from poot_b200.oracle.runner import random_weights_f32
    from poot_b200.text.codec import ByteTokenizer
    for labels in (0, 1):
        cfg = EncoderConfig(n_layers=2, hidden=128, n_heads=4, ffn=256, vocab=300, max_position=64, labels=labels)
        model = EncoderModel(cfg)
        w = random_weights_f32(model, seed=3, std=0.08)
        for k in w:
            if k.endswith("_bias"):
                w[k] = (0.1 * np.random.default_rng(len(k)).standard_normal(w[k].shape)).astype(np.float32)
        w = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}
        tk = PairTokenizer(ByteTokenizer(cfg.vocab), cfg.vocab - 2, cfg.vocab - 1)
        rng = np.random.default_rng(1)
        ids = [rng.integers(3, 290, n).tolist() for n in (21, 5, 33)]          # ragged, across K/V block boundaries
        types = [[0] * (len(x) // 2) + [1] * (len(x) - len(x) // 2) for x in ids]
        host = Embedder(model, w, tk)
        want = host.forward(ids, types)
        with emulated_kernels():
            dev = Embedder(model, w, tk).to_device("cpu", max_tokens=128, max_rows=4)
            got = dev.forward(ids, types)
            assert dev.engine.launches == 6 + 13 * cfg.n_layers
            if labels:
                assert got.shape == (3, 1) and np.abs(got - want).max() < 0.03 * max(1.0, np.abs(want).max())
                continue
            for r, x in enumerate(ids):
                err = np.abs(got[r, :len(x)] - want[r, :len(x)]).max()
                assert err < 0.03 * max(1.0, np.abs(want[r, :len(x)]).max()), (r, err)
            e_dev, e_host = dev.embed_ids(ids), host.embed_ids(ids)
            assert np.abs((e_dev * e_host).sum(-1) - 1.0).max() < 2e-3          # the same directions
            with pytest.raises(ValueError, match="exceed"):
                dev.forward([list(range(3, 60))] * 3)


def test_vision_engine_matches_the_graph_oracle():
    """The SmolVLM vision tower and connector on the device engine's kernels (restated on the host) against the traced
    tower evaluated by the oracle: patch GEMM + position rows, pre-norm blocks with whole-frame attention, final norm,
    pixel shuffle, projection."""
    from poot_b200.models.vision import VisionConfig, VisionTower, patchify, position_ids
    from poot_b200.oracle.eval import EvalOptions, eval_graph
    from poot_b200.runtime.vision_engine import VisionEngine
    cfg = VisionConfig(hidden=128, ffn=256, n_layers=2, n_heads=4, image_size=48, patch=8, scale=2, text_hidden=96)
    tower = VisionTower(cfg)
    rng = np.random.default_rng(0)
    w = {}
    for k, shape in tower.weight_shapes().items():
        v = rng.standard_normal(shape) * (0.1 if k.endswith("_bias") else 0.06)
        if k.endswith("norm"):
            v = 1.0 + 0.1 * rng.standard_normal(shape)
        w[k] = torch.from_numpy(v.astype(np.float32)).to(torch.bfloat16).float().numpy()
    pixels = rng.standard_normal((3, 3, 48, 48)).astype(np.float32)
    g = tower.trace(3)
    inputs = {"patches": patchify(pixels, 8), "pos_ids": np.tile(position_ids(cfg, 6, 6)[None], (3, 1))}
    inputs.update({i.name: w[i.name] for i in g.inputs if i.storage == "const"})
    want = eval_graph(g, inputs, EvalOptions(matmul_precision="exact")).outputs["image_rows"]
    with emulated_kernels():
        eng = VisionEngine(cfg, {k: torch.from_numpy(v) for k, v in w.items()}, "cpu", max_frames=4)
        got = eng.forward(pixels).float().numpy()
        assert eng.launches == 4 + 13 * cfg.n_layers + 3
        with pytest.raises(ValueError, match="frames exceed"):
            eng.forward(np.zeros((5, 3, 48, 48), np.float32))
    assert got.shape == want.shape == (3 * 9, 96)
    assert np.abs(got - want).max() < 0.03 * max(1.0, np.abs(want).max())
    with pytest.raises(ValueError, match="multiples of 32"):
        VisionEngine(VisionConfig(hidden=48, n_heads=4), {}, "cpu")


def test_guided_steps_are_cut_at_the_late_input_point():
    """A guided sequence on the device step engine: the mask arrives as a callable, the engine launches the model body,
    builds and binds the mask, then launches the sampler suffix; the constrained output is what the eager mask gives."""
    from poot_b200 import LLM, SamplingParams
    from poot_b200.text.guided import build_constraint
    over = dict(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512, max_position=256)

    def run(late: bool):
        llm = LLM.random("tiny-llama", device="cpu", rows=2, max_seq=64, prefill_chunk=16, num_blocks=16, std=0.08, **over)
        d = llm.driver
        inner = d.engine.inner
        inner.late_inputs = late
        order = []
        e = inner.e
        body, sample = e.forward, e._sample

        def spy_forward(shape):
            order.append("forward:" + str(e._stage))
            return body(shape)

        e.forward = spy_forward
        g = build_constraint({"choice": ["yes", "no", "maybe"]}, llm.tokenizer, d.eos_token)
        mask = g.mask

        def spy_mask(vocab):
            order.append("mask")
            return mask(vocab)

        g.mask = spy_mask
        sid = d.open(llm.tokenizer.encode("answer:"), SamplingParams(max_tokens=8), guided=g)
        out = []
        for _ in range(8):
            r = d.step([sid])[0]
            d.commit(sid, [r.token])
            if d.finished(sid, r.token):
                if r.token != d.eos_token:
                    out.append(r.token)
                break
            out.append(r.token)
        d.release(sid)
        return llm.tokenizer.decode(out), order, inner.late_steps

    with emulated_kernels():
        text_late, order_late, n_late = run(True)
        text_eager, order_eager, n_eager = run(False)
    assert text_late == text_eager and text_late in ("yes", "no", "maybe")
    assert n_late > 0 and n_eager == 0
    assert order_late[:3] == ["forward:body", "mask", "forward:suffix"]       # the mask is built between the stages
    assert order_eager[:2] == ["mask", "forward:None"]
