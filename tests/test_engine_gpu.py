"""Whole-model checks of the device engine against the PyTorch fp32 restatement of the stack."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(cfg, batch, max_len, max_tokens, use_graphs=True, seed=0):
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_weights
    w = random_weights(cfg, "cuda", seed=seed, std=0.05)
    bps = (max_len + 15) // 16
    eng = DecoderEngine(w, num_blocks=batch * bps, max_seqs=batch, max_tokens=max_tokens, max_blocks_per_seq=bps,
                        use_graphs=use_graphs)
    return w, eng, FixedBatchSession(eng, batch, max_len)


def _small_cfg(**kw):
    from poot_b200.models.config import DecoderConfig
    base = dict(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=688, vocab=2048, max_position=512)
    base.update(kw)
    return DecoderConfig(**base)


@pytest.mark.parametrize("graphs", [False, True])
def test_prefill_logits_match_reference(graphs):
    from poot_b200.oracle.torch_ref import forward_logits
    from poot_b200.ops import cuda_ops as K
    cfg = _small_cfg()
    w, eng, sess = _engine(cfg, batch=2, max_len=64, max_tokens=64, use_graphs=graphs)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (2, 24), generator=g, dtype=torch.int32)
    picked = sess.prefill_fast(prompts)
    K.check_status()
    for b in range(2):
        ref = forward_logits(w, prompts[b].cuda())[-1]
        got = eng.logits[b]
        assert torch.isfinite(got).all()
        err = (got - ref).abs().max().item()
        assert err < 0.05 * max(1.0, ref.abs().max().item()), err
        assert picked[b, 1] == -1
        top2 = torch.topk(ref, 2).values
        if (top2[0] - top2[1]) > 0.05:
            assert picked[b, 0] == int(ref.argmax())


def test_decode_steps_equal_prefill():
    """Decoding token by token through the paged cache gives the logits of a one-shot prefill."""
    cfg = _small_cfg(n_heads=8, n_kv_heads=2, head_dim=128, hidden=512, ffn=1024)
    w, eng, sess = _engine(cfg, batch=1, max_len=64, max_tokens=64)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (1, 20), generator=g, dtype=torch.int32)
    sess.prefill_fast(toks)
    full = eng.logits[0].clone()
    w2, eng2, sess2 = _engine(cfg, batch=1, max_len=64, max_tokens=64)
    sess2.prefill_fast(toks[:, :12])
    for t in range(12, 20):
        sess2.decode([int(toks[0, t])])
    err = (eng2.logits[0] - full).abs().max().item()
    assert err < 0.03 * max(1.0, full.abs().max().item()), err


def test_decode_batch64_uses_tensor_core_path():
    from poot_b200.oracle.torch_ref import forward_logits
    from poot_b200.ops import cuda_ops as K
    cfg = _small_cfg(hidden=512, ffn=1536, n_heads=8, n_kv_heads=2, head_dim=64)
    B = 64
    w, eng, sess = _engine(cfg, batch=B, max_len=32, max_tokens=B * 8)
    g = torch.Generator().manual_seed(2)
    prompts = torch.randint(0, cfg.vocab, (B, 8), generator=g, dtype=torch.int32)
    sess.prefill_fast(prompts)
    nxt = torch.randint(0, cfg.vocab, (B,), generator=g, dtype=torch.int32)
    sess.decode(nxt.tolist())
    K.check_status()
    for b in (0, 31, 63):
        seq = torch.cat([prompts[b], nxt[b:b + 1]]).cuda()
        ref = forward_logits(w, seq)[-1]
        err = (eng.logits[b] - ref).abs().max().item()
        assert err < 0.05 * max(1.0, ref.abs().max().item()), (b, err)


def test_chained_decode_matches_stepwise():
    cfg = _small_cfg()
    w, eng, sess = _engine(cfg, batch=2, max_len=64, max_tokens=64)
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, cfg.vocab, (2, 10), generator=g, dtype=torch.int32)
    first = sess.prefill_fast(prompts)[:, 0].tolist()
    toks = list(first)
    stepwise = []
    for _ in range(6):
        toks = sess.decode(toks)[:, 0].tolist()
        stepwise.append(list(toks))
    w2, eng2, sess2 = _engine(cfg, batch=2, max_len=64, max_tokens=64)
    first2 = sess2.prefill_fast(prompts)[:, 0].tolist()
    assert first2 == first
    sess2.decode_chain(first2, steps=6)
    torch.cuda.synchronize()
    assert eng2.picked[:2, 0].tolist() == stepwise[-1]


def test_qk_norm_and_window_model():
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = _small_cfg(qk_norm=True, sliding_window=8)
    w, eng, sess = _engine(cfg, batch=1, max_len=64, max_tokens=64)
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, cfg.vocab, (1, 30), generator=g, dtype=torch.int32)
    sess.prefill_fast(toks)
    ref = forward_logits(w, toks[0].cuda())[-1]
    err = (eng.logits[0] - ref).abs().max().item()
    assert err < 0.05 * max(1.0, ref.abs().max().item()), err


@pytest.mark.xfail(strict=False, reason="device path written without a device at hand: checked on the CPU against "
                                        "the oracle only (tests/test_families.py); must not hide the suite behind it")
@pytest.mark.parametrize("kw", [dict(attn_bias=True, tie_embeddings=True),                      # qwen2-style
                                dict(embed_scale=12.0, residual_scale=0.22, logit_scale=0.125),   # granite-style
                                dict(head_dim=128, n_heads=4, n_kv_heads=1, hidden=512, attn_bias=True)])
def test_bias_and_constant_multipliers(kw):
    """q/k/v bias and the embedding scale are applied at run time, residual and logit scales are folded into the weights."""
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = _small_cfg(**kw)
    w, eng, sess = _engine(cfg, batch=2, max_len=64, max_tokens=64)
    g = torch.Generator().manual_seed(6)
    toks = torch.randint(0, cfg.vocab, (2, 21), generator=g, dtype=torch.int32)
    sess.prefill_fast(toks)
    for b in range(2):
        ref = forward_logits(w, toks[b].cuda())[-1]
        err = (eng.logits[b] - ref).abs().max().item()
        assert err < 0.05 * max(1.0, ref.abs().max().item()), (b, err)
    nxt = torch.randint(0, cfg.vocab, (2,), generator=g, dtype=torch.int32)
    sess.decode(nxt.tolist())
    ref = forward_logits(w, torch.cat([toks[0], nxt[:1]]).cuda())[-1]
    err = (eng.logits[0] - ref).abs().max().item()
    assert err < 0.05 * max(1.0, ref.abs().max().item()), err


@pytest.mark.xfail(strict=False, reason="new device paths: not yet run on a device")
@pytest.mark.parametrize("name", ["gemma2", "gemma3", "olmo2", "olmoe", "smollm3-nope-layer", "granite", "minimax_m2", "qwen3_5", "qwen3next", "deepseek2", "deepseek3", "gpt_oss", "mpt", "bloom", "nemotron_h"])
def test_family_blocks_match_the_graph_oracle(name):
    """The device twin of the host-emulated check: sandwich / post norms, GeGLU, soft caps, two rope bases,
    projection-wide q/k norms and layers without rope on the real kernels, against the graph oracle."""
    import numpy as np
    from test_engine_emulated import HF_BASE, HF_FAMILIES
    from poot_b200.models.registry import Registry
    from poot_b200.ops import cuda_ops as K
    from poot_b200.oracle.runner import OracleSession, random_weights_f32
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import from_named_tensors
    model = Registry.builtin().resolve_hf(HF_FAMILIES[name] if name in ("mpt", "bloom") else {**HF_BASE, **HF_FAMILIES[name]})
    cfg = model.cfg
    w = random_weights_f32(model, seed=2, std=0.08)
    w = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}
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
    ref = torch.from_numpy(OracleSession(model, w, capacity=32).step(toks))[0]
    dw = from_named_tensors(cfg, named, "cuda")
    eng = DecoderEngine(dw, num_blocks=4, max_seqs=1, max_tokens=32, max_blocks_per_seq=2)
    s = FixedBatchSession(eng, 1, 32)
    s.prefill_fast(torch.from_numpy(toks[:, :20]).int())
    for t in range(20, 23):
        s.decode([int(toks[0, t])])
    K.check_status()
    err = (eng.logits[0].cpu() - ref).abs().max().item()
    assert err < 0.03 * max(1.0, ref.abs().max().item()), (name, err)


@pytest.mark.xfail(strict=False, reason="per-row adapters through the grouped GEMM: not yet run on a device")
def test_rows_with_and_without_a_resident_adapter():
    """Device twin of the host-emulated adapter check: one decode step of three rows (adapter a, adapter b, none)."""
    import numpy as np
    from test_engine_emulated import adapter_roles, make_adapter, merged_weights
    from poot_b200.oracle.torch_ref import forward_logits
    from poot_b200.ops import cuda_ops as K
    from poot_b200.runtime.engine import StepShape
    cfg = _small_cfg()
    w, eng, sess = _engine(cfg, batch=3, max_len=64, max_tokens=96, use_graphs=False)
    bank = eng.enable_adapters(slots=4, max_rank=8)
    rng = np.random.default_rng(0)
    every = adapter_roles(cfg)
    ads = [make_adapter(cfg, rng, "a", 8, every), make_adapter(cfg, rng, "b", 4, {"attn_q": every["attn_q"], "ffn_down": every["ffn_down"]})]
    slots = [bank.load(ads[0]), bank.load(ads[1]), -1]
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (3, 17), generator=g, dtype=torch.int32)
    sess.prefill_fast(prompts)           # base-model prefill only fills positions; the checked step recomputes row by row below
    refs = [merged_weights(cfg, w, ads[0]), merged_weights(cfg, w, ads[1]), w]
    # a fresh session so that every row's K/V is computed under its own adapter
    w2, eng2, s2 = _engine(cfg, batch=3, max_len=64, max_tokens=96, use_graphs=False)
    bank2 = eng2.enable_adapters(slots=4, max_rank=8)
    for a in ads:
        bank2.load(a)
    T = 3 * 17
    bank2.bind_rows(np.repeat(np.array(slots, np.int32), 17), T)
    B, L = prompts.shape
    pos = torch.arange(L, dtype=torch.int32).repeat(B)
    seq = torch.arange(B, dtype=torch.int32).repeat_interleave(L)
    s2.h_tokens[:T] = prompts.reshape(-1)
    s2.h_pos[:T], s2.h_seq[:T] = pos, seq
    blk = s2.block_tables_host[seq.long(), (pos // 16).long()]
    s2.h_slots[:T] = blk * 16 + pos % 16
    s2.h_ctx[:T] = pos + 1
    s2.h_lidx[:B] = torch.arange(B, dtype=torch.int64) * L + (L - 1)
    s2.lengths = [L] * B
    s2._step(StepShape(T, B, 0, lora=True))
    K.check_status()
    for b in range(3):
        ref = forward_logits(refs[b], prompts[b].cuda())[-1]
        err = (eng2.logits[b] - ref).abs().max().item()
        assert err < 0.05 * max(1.0, ref.abs().max().item()), (b, err)


@pytest.mark.xfail(strict=False, reason="the encoder program (BERT) on the device engine: not yet run on a device")
def test_encoder_engine_matches_the_graph_oracle_on_the_device():
    import numpy as np
    from poot_b200.embed import Embedder, PairTokenizer
    from poot_b200.models.encoder import EncoderConfig, EncoderModel
    from poot_b200.oracle.runner import random_weights_f32
    from poot_b200.text.codec import ByteTokenizer
    cfg = EncoderConfig(n_layers=2, hidden=384, n_heads=12, ffn=1536, vocab=1000, max_position=128)
    model = EncoderModel(cfg)
    w = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in random_weights_f32(model, seed=3, std=0.05).items()}
    tk = PairTokenizer(ByteTokenizer(cfg.vocab), cfg.vocab - 2, cfg.vocab - 1)
    rng = np.random.default_rng(1)
    ids = [rng.integers(3, 990, n).tolist() for n in (21, 5, 97, 64)]
    want = Embedder(model, w, tk).forward(ids)
    got = Embedder(model, w, tk).to_device("cuda", max_tokens=256, max_rows=4).forward(ids)
    for r, x in enumerate(ids):
        err = np.abs(got[r, :len(x)] - want[r, :len(x)]).max()
        assert err < 0.03 * max(1.0, np.abs(want[r, :len(x)]).max()), (r, err)


@pytest.mark.xfail(strict=False, reason="the vision tower program on the device engine: not yet run on a device")
def test_vision_engine_matches_the_graph_oracle_on_the_device():
    import numpy as np
    from poot_b200.models.vision import VisionConfig, VisionTower, patchify, position_ids
    from poot_b200.oracle.eval import EvalOptions, eval_graph
    from poot_b200.runtime.vision_engine import VisionEngine
    cfg = VisionConfig(hidden=256, ffn=512, n_layers=2, n_heads=4, image_size=128, patch=16, scale=4, text_hidden=192)
    tower = VisionTower(cfg)
    rng = np.random.default_rng(0)
    w = {}
    for k, shape in tower.weight_shapes().items():
        v = 1.0 + 0.1 * rng.standard_normal(shape) if k.endswith("norm") else rng.standard_normal(shape) * 0.05
        w[k] = torch.from_numpy(v.astype(np.float32)).to(torch.bfloat16).float().numpy()
    pixels = rng.standard_normal((2, 3, 128, 128)).astype(np.float32)
    g = tower.trace(2)
    inputs = {"patches": patchify(pixels, 16), "pos_ids": np.tile(position_ids(cfg, 8, 8)[None], (2, 1))}
    inputs.update({i.name: w[i.name] for i in g.inputs if i.storage == "const"})
    want = eval_graph(g, inputs, EvalOptions(matmul_precision="exact")).outputs["image_rows"]
    got = VisionEngine(cfg, {k: torch.from_numpy(v) for k, v in w.items()}, "cuda", max_frames=2).forward(pixels).float().cpu().numpy()
    assert np.abs(got - want).max() < 0.03 * max(1.0, np.abs(want).max())
