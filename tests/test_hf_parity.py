"""Golden parity with the Hugging Face implementations, on the CPU.

For every supported family a tiny randomly initialised ``transformers`` model is saved as a checkpoint directory
(``config.json`` + safetensors), loaded through this package's own path (registry -> name tables -> weight store) and
evaluated by the graph oracle; the logits of every position must equal the ``transformers`` forward pass to float
precision.  That pins, independently of this package's own restatements, the header parsing of each family, its
tensor-name table (fused projections, stacked experts, per-head interleaving) and the semantics of its block: norm
placement, activations, biases, ALiBi, sliding windows per layer, two rotary bases, soft caps, attention sinks,
router variants, shared experts, group-limited routing and multi-head latent attention."""
import numpy as np
import pytest

transformers = pytest.importorskip("transformers")
torch = pytest.importorskip("torch")

from poot_b200.driver.handle import ModelHandle          # noqa: E402
from poot_b200.models.model import StepSpec              # noqa: E402
from poot_b200.oracle.runner import OracleSession        # noqa: E402

BASE = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
            intermediate_size=96, vocab_size=200, max_position_embeddings=128)
MLA = dict(n_routed_experts=8, num_experts_per_tok=3, moe_intermediate_size=32, first_k_dense_replace=1, kv_lora_rank=24,
           qk_rope_head_dim=8, qk_nope_head_dim=16, v_head_dim=12, num_key_value_heads=4, head_dim=8)
CASES = {
    "llama": dict(model_type="llama", rms_norm_eps=1e-5),
    "llama-biases": dict(model_type="llama", attention_bias=True, mlp_bias=True),
    "mistral-window": dict(model_type="mistral", sliding_window=8),
    "mixtral": dict(model_type="mixtral", num_local_experts=4, num_experts_per_tok=2),
    "qwen2": dict(model_type="qwen2", tie_word_embeddings=True),
    "qwen3": dict(model_type="qwen3"),
    "olmo2": dict(model_type="olmo2"),
    "phi3": dict(model_type="phi3", pad_token_id=0),
    "smollm3-nope-layer": dict(model_type="smollm3", pad_token_id=0, no_rope_layers=[1, 0]),
    "granite": dict(model_type="granite", embedding_multiplier=12.0, residual_multiplier=0.22, logits_scaling=8.0,
                    attention_multiplier=0.2),
    "granitemoe": dict(model_type="granitemoe", num_local_experts=4, num_experts_per_tok=2, intermediate_size=32,
                       embedding_multiplier=3.0, residual_multiplier=0.5, logits_scaling=4.0, attention_multiplier=0.3),
    "qwen3moe": dict(model_type="qwen3_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True),
    "olmoe": dict(model_type="olmoe", num_experts=4, num_experts_per_tok=2, intermediate_size=32),
    "gemma2": dict(model_type="gemma2", query_pre_attn_scalar=24, sliding_window=6, attn_logit_softcapping=5.0,
                   final_logit_softcapping=3.0),
    "gemma3": dict(model_type="gemma3_text", query_pre_attn_scalar=24, sliding_window=6, num_hidden_layers=3,
                   layer_types=["sliding_attention", "sliding_attention", "full_attention"]),
    # latent attention behind the sparse attention indexer: every query keeps its 5 best-scored keys (DeepSeek-V3.2's
    # mechanism; six indexer heads keep exact zero ties of the rectified scores out of the cut)
    "glm_moe_dsa": dict(model_type="glm_moe_dsa", num_hidden_layers=3, q_lora_rank=32, kv_lora_rank=24, qk_rope_head_dim=8,
                        qk_nope_head_dim=16, v_head_dim=12, num_key_value_heads=4, head_dim=8, n_routed_experts=8,
                        num_experts_per_tok=3, moe_intermediate_size=32, n_shared_experts=1, n_group=2, topk_group=1,
                        mlp_layer_types=["dense", "sparse", "sparse"], index_topk=5, index_n_heads=6, index_head_dim=16,
                        routed_scaling_factor=2.5, pad_token_id=0, _scale=3.0),
    # gemma4: head width by layer type, proportional rope, scores without a scale, weightless v norm, layer scalars ...
    "gemma4": dict(model_type="gemma4_text", num_hidden_layers=4, global_head_dim=32, sliding_window=6, vocab_size_per_layer_input=200,
                   layer_types=["sliding_attention", "full_attention"] * 2, hidden_size_per_layer_input=0, pad_token_id=0, _scale=2.0),
    # ... per-layer embeddings, the last two layers attending over the K/V of layers 0 / 1, double-width FFNs there
    "gemma4-per-layer-embeddings-shared-kv": dict(
        model_type="gemma4_text", num_hidden_layers=4, global_head_dim=32, sliding_window=6, vocab_size_per_layer_input=200,
        layer_types=["sliding_attention", "full_attention"] * 2, hidden_size_per_layer_input=8, num_kv_shared_layers=2,
        use_double_wide_mlp=True, pad_token_id=0, _scale=2.0),
    # ... full-attention layers whose value is the key projection, on one K/V head; capped logits
    "gemma4-value-is-key": dict(model_type="gemma4_text", num_hidden_layers=4, global_head_dim=32, sliding_window=6,
                                vocab_size_per_layer_input=200, layer_types=["sliding_attention", "full_attention"] * 2,
                                hidden_size_per_layer_input=0, attention_k_eq_v=True, num_global_key_value_heads=1,
                                final_logit_softcapping=30.0, pad_token_id=0, _scale=2.0),
    # ... a dense FFN plus routed experts in every layer, the router on the un-normed residual, per-expert gate scales
    "gemma4-moe": dict(model_type="gemma4_text", num_hidden_layers=4, global_head_dim=32, sliding_window=6,
                       vocab_size_per_layer_input=200, layer_types=["sliding_attention", "full_attention"] * 2,
                       hidden_size_per_layer_input=0, enable_moe_block=True, num_experts=4, top_k_experts=2,
                       moe_intermediate_size=48, pad_token_id=0, _scale=2.0),
    "mpt": dict(model_type="mpt", d_model=64, n_heads=4, n_layers=2, vocab_size=200, max_seq_len=128),
    "mpt-6-heads": dict(model_type="mpt", d_model=96, n_heads=6, n_layers=2, vocab_size=200, max_seq_len=128),
    "bloom": dict(model_type="bloom", hidden_size=64, n_head=4, n_layer=2, vocab_size=200),
    "bloom-6-heads": dict(model_type="bloom", hidden_size=96, n_head=6, n_layer=2, vocab_size=200),
    "gpt_oss": dict(model_type="gpt_oss", num_local_experts=4, num_experts_per_tok=2, intermediate_size=32, sliding_window=6,
                    layer_types=["sliding_attention", "full_attention"],
                    rope_parameters={"rope_type": "default", "rope_theta": 10000.0}),
    "minimax_m2": dict(model_type="minimax_m2", num_local_experts=4, num_experts_per_tok=2, intermediate_size=32),
    "deepseek2": dict(model_type="deepseek_v2", q_lora_rank=None, n_shared_experts=2, **MLA),
    "deepseek3": dict(model_type="deepseek_v3", q_lora_rank=32, n_shared_experts=1, n_group=4, topk_group=2, **MLA),
    # Mamba2 + attention + routed non-gated experts.  The library's float32 chunked scan loses a few 1e-6 where it
    # carries state across a chunk boundary (positions past the first chunk), which the later blocks amplify; one
    # chunk covers the test sequence so the comparison is against its exact path.
    "nemotron_h": dict(model_type="nemotron_h", layers_block_type=["mamba", "moe", "attention", "moe"], mamba_num_heads=4,
                       mamba_head_dim=16, ssm_state_size=8, n_groups=2, conv_kernel=4, chunk_size=16, time_step_min=1e-7,
                       n_routed_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                       moe_shared_expert_intermediate_size=48),
    "qwen3next": dict(model_type="qwen3_next", layer_types=["linear_attention", "full_attention"], linear_num_value_heads=4,
                      linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
                      num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=48,
                      _tol=1e-4),
    "qwen3_5": dict(model_type="qwen3_5_text", layer_types=["linear_attention", "full_attention"], linear_num_value_heads=4,
                    linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4, _tol=1e-4),
}
OWN_DIMS = ("mpt", "bloom")      # families whose headers do not use the llama field names


def build(case: dict):
    from transformers import AutoConfig, AutoModelForCausalLM
    over = {k: v for k, v in case.items() if not k.startswith("_")}
    mt = over.pop("model_type")
    d = over if mt in OWN_DIMS else {**BASE, **over}
    cfg = AutoConfig.for_model(mt, **d)
    torch.manual_seed(0)
    m = AutoModelForCausalLM.from_config(cfg, attn_implementation="eager").float().eval()
    with torch.no_grad():          # default initialisation is too tame to show a wrong norm or a wrong bias
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
            else:
                p.mul_(case.get("_scale", 4.0))
    return m, d["vocab_size"]


@pytest.mark.parametrize("name", sorted(CASES))
def test_logits_equal_the_hugging_face_forward(name, tmp_path):
    m, vocab = build(CASES[name])
    toks = torch.randint(0, vocab, (1, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(toks).logits[0].numpy()
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    h = ModelHandle.load(str(tmp_path))
    sess = OracleSession(h.model, h.oracle_weights(), capacity=32)
    sess._graph = lambda T, embeds=False: h.model.trace(StepSpec(rows=1, tokens=T, capacity=32, logit_rows="all"))
    got = sess.step(toks.numpy()).reshape(ref.shape)
    assert np.isfinite(got).all()
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err < CASES[name].get("_tol", 2e-5), err


@pytest.mark.parametrize("name", ["llama", "gemma3", "bloom", "deepseek3", "gpt_oss", "qwen3next", "nemotron_h",
                                  "gemma4-per-layer-embeddings-shared-kv", "glm_moe_dsa"])
def test_driver_over_the_oracle_engine_generates_what_hugging_face_generates(name, tmp_path):
    """End to end on the host: checkpoint directory -> ``LLM.oracle`` -> driver (paged K/V through block tables,
    chunked prefill, two sequences in flight) gives the greedy continuation ``transformers`` gives."""
    from poot_b200 import LLM, SamplingParams
    m, vocab = build(CASES[name])
    m.generation_config.eos_token_id = None
    m.generation_config.pad_token_id = 0
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    llm = LLM.oracle(str(tmp_path), rows=2, max_seq=64, num_blocks=16, prefill_chunk=16)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, vocab, (1, n), generator=g) for n in (37, 5)]
    want = []
    for p in prompts:
        with torch.no_grad():
            out = m.generate(p, max_new_tokens=6, do_sample=False, eos_token_id=None)
        want.append(out[0, p.shape[1]:].tolist())
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    drv = llm.driver
    ids = [drv.open(p[0].tolist(), sp) for p in prompts]
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
    assert [got[i] for i in ids] == want


def test_cli_generates_from_a_checkpoint_on_the_oracle_backend(tmp_path):
    """``generate -m DIR --backend oracle`` runs a checkpoint of a family the device program does not cover."""
    import io
    from poot_b200.cli.generate import parse_generate, run_generate
    m, vocab = build(CASES["gemma2"])
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    out = io.StringIO()
    r = run_generate(parse_generate(["-m", str(tmp_path), "--backend", "oracle", "-p", "ab", "-n", "4", "--temp", "0",
                                     "--no-chat-template", "--ignore-eos"]), out=out)
    assert r["generated"] == 4


# ---- encoders --------------------------------------------------------------------------------------------------
BERT = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, vocab_size=300,
            max_position_embeddings=64, type_vocab_size=2)


def _bert(cls, tmp_path, **kw):
    from transformers import BertConfig
    torch.manual_seed(0)
    m = cls(BertConfig(**BERT, **kw)).float().eval()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
            else:
                p.mul_(3.0)
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    return m


def test_bert_hidden_states_equal_hugging_face_and_ignore_padding(tmp_path):
    from transformers import BertModel
    from poot_b200.embed import Embedder
    m = _bert(BertModel, tmp_path)
    emb = Embedder.load(str(tmp_path))
    g = torch.Generator().manual_seed(3)
    a, b = torch.randint(1, 300, (1, 11), generator=g), torch.randint(1, 300, (1, 5), generator=g)
    with torch.no_grad():
        ra = m(a).last_hidden_state[0].numpy()
        rb = m(b).last_hidden_state[0].numpy()
    hid = emb.forward([a[0].tolist(), b[0].tolist()])          # one right-padded batch
    assert np.abs(hid[0, :11] - ra).max() < 1e-4 * np.abs(ra).max()
    assert np.abs(hid[1, :5] - rb).max() < 1e-4 * np.abs(rb).max()
    vec = emb.embed_ids([a[0].tolist(), b[0].tolist()])
    want = ra.mean(0) / np.linalg.norm(ra.mean(0))
    assert np.allclose(vec[0], want, atol=1e-5) and abs(np.linalg.norm(vec[1]) - 1) < 1e-5


def test_bert_cross_encoder_scores_and_http_routes(tmp_path):
    import json
    import urllib.request
    from transformers import BertForSequenceClassification
    from poot_b200.embed import Embedder, EmbedEngine
    from poot_b200.serve.config import ServeConfig
    from poot_b200.serve.http import Server, ServerState
    from poot_b200.serve.metrics import Metrics
    m = _bert(BertForSequenceClassification, tmp_path, num_labels=1)
    emb = Embedder.load(str(tmp_path))
    assert emb.cfg.labels == 1
    ids, types = emb.tk.encode("what is a kernel", "a function that runs on the device")
    with torch.no_grad():
        want = m(torch.tensor([ids]), token_type_ids=torch.tensor([types])).logits[0, 0].item()
    scores, _ = emb.rerank("what is a kernel", ["a function that runs on the device", "bread"])
    assert abs(float(scores[0]) - want) < 1e-4 * max(1.0, abs(want))
    cfg = ServeConfig(model=str(tmp_path), addr="127.0.0.1:0")
    server = Server(ServerState(EmbedEngine(emb, Metrics()), cfg, "tiny-cross-encoder", family="bert"))
    server.start()
    try:
        def post(path, body):
            req = urllib.request.Request(f"http://127.0.0.1:{server.port}{path}", json.dumps(body).encode(),
                                         {"Content-Type": "application/json"})
            try:
                with urllib.request.urlopen(req, timeout=30) as r:
                    return r.status, json.loads(r.read())
            except urllib.error.HTTPError as e:
                return e.code, json.loads(e.read())
        st, body = post("/v1/rerank", {"query": "what is a kernel", "documents": ["a function that runs on the device", {"text": "bread"}],
                                       "return_documents": True})
        assert st == 200 and len(body["results"]) == 2
        top = body["results"][0]
        assert abs(top["relevance_score"] - float(scores[top["index"]])) < 1e-6 and "text" in top["document"]
        assert body["results"][0]["relevance_score"] >= body["results"][1]["relevance_score"]
        st, body = post("/v1/embeddings", {"input": "x"})
        assert st == 400 and "classifier" in body["error"]["message"]
        st, body = post("/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}]})
        assert st == 400 and "encoder" in body["error"]["message"]
    finally:
        server.shutdown()


def test_embeddings_route_and_cli(tmp_path, capsys):
    import base64
    import json
    import urllib.request
    from transformers import BertModel
    from poot_b200.cli.__main__ import main
    from poot_b200.embed import Embedder, EmbedEngine
    from poot_b200.serve.config import ServeConfig
    from poot_b200.serve.http import Server, ServerState
    from poot_b200.serve.metrics import Metrics
    _bert(BertModel, tmp_path)
    emb = Embedder.load(str(tmp_path))
    server = Server(ServerState(EmbedEngine(emb, Metrics()), ServeConfig(model=str(tmp_path), addr="127.0.0.1:0"), "tiny-bert", family="bert"))
    server.start()
    try:
        def post(body):
            req = urllib.request.Request(f"http://127.0.0.1:{server.port}/v1/embeddings", json.dumps(body).encode(),
                                         {"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=30) as r:
                return json.loads(r.read())
        r = post({"input": ["alpha", "beta gamma"], "model": "tiny-bert"})
        want, n = emb.embed(["alpha", "beta gamma"])
        assert r["usage"]["prompt_tokens"] == n and len(r["data"]) == 2
        assert np.allclose(r["data"][1]["embedding"], want[1], atol=1e-6)
        r64 = post({"input": "alpha", "encoding_format": "base64", "dimensions": 16})
        v = np.frombuffer(base64.b64decode(r64["data"][0]["embedding"]), "<f4")
        assert v.shape == (16,) and np.allclose(v, want[0][:16], atol=1e-6)
    finally:
        server.shutdown()
    assert main(["embed", "similarity", str(tmp_path), "alpha", "alpha", "zz top"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert lines[0].startswith("pooling") and lines[1].startswith("+1.000") and len(lines) == 3
    assert main(["embed", "cross", str(tmp_path), "q", "d"]) == 2      # not a cross-encoder


def test_qwen3_5_checkpoint_on_the_emulated_device_engine_generates_what_hugging_face_generates(tmp_path):
    """The whole device path for a hybrid checkpoint - loader, fused layouts, gated delta net and gated attention
    layers, per-sequence conv / state carry through chunked prefill and decode, two sequences in flight - with the
    kernels restated on the host."""
    from poot_b200 import LLM, SamplingParams
    from poot_b200.utils.kernel_emulation import emulated_kernels
    case = dict(CASES["qwen3_5"], head_dim=64, linear_key_head_dim=64, linear_value_head_dim=64, hidden_size=128,
                rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.5, "rope_type": "default"})
    m, vocab = build(case)
    m.generation_config.eos_token_id = None
    m.generation_config.pad_token_id = 0
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, vocab, (1, n), generator=g) for n in (37, 5)]
    want = []
    for p in prompts:
        with torch.no_grad():
            out = m.generate(p, max_new_tokens=5, do_sample=False, eos_token_id=None)
        want.append(out[0, p.shape[1]:].tolist())
    with emulated_kernels():
        llm = LLM.load(str(tmp_path), device="cpu", rows=2, max_seq=64, prefill_chunk=16, num_blocks=16)
        assert llm.cfg.device_gaps() == [] and llm.driver.prefix is None
        sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
        drv = llm.driver
        ids = [drv.open(p[0].tolist(), sp) for p in prompts]
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
    # bf16 weights and activations on the engine side: compare where the reference's top two logits are not a near tie
    agree = sum(a == b for i, w_ in zip(ids, want) for a, b in zip(got[i], w_))
    assert agree >= 8, (got, want)


DEVICE_CASES = {
    # the parity cases at widths the device kernels take (head widths that are multiples of 32)
    "gemma2": dict(head_dim=32, hidden_size=128),
    "gemma3": dict(head_dim=32, hidden_size=128),
    "olmo2": dict(head_dim=32, hidden_size=128),
    "granitemoe": dict(head_dim=32, hidden_size=128),
    "gpt_oss": dict(head_dim=32, hidden_size=128),
    "minimax_m2": dict(head_dim=32, hidden_size=128),
    "bloom": dict(hidden_size=128, n_head=4),
    "mpt": dict(d_model=128, n_heads=4),
    "deepseek3": dict(hidden_size=128, qk_rope_head_dim=32, qk_nope_head_dim=32, v_head_dim=32, head_dim=32),
    # latent attention behind the sparse indexer on the device program: index keys in their own paged pool, scores over the
    # visible keys, exact top-k selection, attention over the kept positions only
    "glm_moe_dsa": dict(hidden_size=128, qk_rope_head_dim=32, qk_nope_head_dim=32, v_head_dim=32, head_dim=32,
                        kv_lora_rank=32, index_head_dim=32),
    "nemotron_h": dict(head_dim=32, hidden_size=128, mamba_head_dim=32),
    "qwen3next": dict(head_dim=32, hidden_size=128, linear_key_head_dim=64, linear_value_head_dim=64,
                      rope_parameters={"rope_theta": 10000.0, "partial_rotary_factor": 0.5, "rope_type": "default"}),
}


@pytest.mark.parametrize("name", sorted(DEVICE_CASES))
def test_checkpoint_through_the_device_loader_and_emulated_engine_follows_hugging_face(name, tmp_path):
    """Checkpoint directory -> ``LLM.load`` (the device loader: fused layouts, biases, folded norm offsets, expert
    stacks, per-family extras) -> the engine's program with the kernels restated on the host -> greedy tokens, against
    ``transformers`` greedy generation.  bf16 weights and activations on the engine side: most tokens must agree (a
    near-tie of the top two logits, or of two router scores, may pick differently)."""
    from poot_b200 import LLM, SamplingParams
    from poot_b200.utils.kernel_emulation import emulated_kernels
    m, vocab = build({**CASES[name], **DEVICE_CASES[name]})
    m.generation_config.eos_token_id = None
    m.generation_config.pad_token_id = 0
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    p = torch.randint(3, vocab, (1, 21), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        want = m.generate(p, max_new_tokens=6, do_sample=False, eos_token_id=None)[0, 21:].tolist()
    with emulated_kernels():
        llm = LLM.load(str(tmp_path), device="cpu", rows=1, max_seq=64, prefill_chunk=16, num_blocks=8)
        assert llm.cfg.device_gaps() == []
        got = llm.generate_tokens(p[0].tolist(), SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    agree = 0
    for a, b in zip(got, want):      # count the common prefix: after a divergence the continuations are different texts
        if a != b:
            break
        agree += 1
    assert agree >= 2, (got, want)


def test_sparse_indexer_on_the_device_program_keeps_the_positions_hugging_face_keeps(tmp_path):
    """First layer of the sparse-attention family through the engine's kernel program (host restatements): the
    positions the indexer keeps for each of 16 prompt rows are exactly the ones ``transformers``' indexer keeps (deeper
    layers see bf16-rounded inputs, where a near-tie at the cut may fall the other way)."""
    from poot_b200 import LLM, SamplingParams
    from poot_b200.utils import kernel_emulation as emu
    m, vocab = build({**CASES["glm_moe_dsa"], **DEVICE_CASES["glm_moe_dsa"]})
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    p = torch.randint(3, vocab, (1, 16), generator=torch.Generator().manual_seed(4))
    kept = {}
    indexer = m.model.layers[0].self_attn.indexer
    forward = indexer.forward

    def spy_hf(*a, **k):
        kept["hf"] = forward(*a, **k)
        return kept["hf"]

    indexer.forward = spy_hf
    with torch.no_grad():
        m(p)
    select = emu.index_select

    def spy_device(scores, row_ctx, sel):
        out = select(scores, row_ctx, sel)
        kept.setdefault("device", sel.clone())
        return out

    emu.index_select = spy_device
    try:
        with emu.emulated_kernels():
            llm = LLM.load(str(tmp_path), device="cpu", rows=1, max_seq=64, prefill_chunk=16, num_blocks=8)
            sid = llm.driver.open(p[0].tolist(), SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True))
            llm.driver.step([sid])
    finally:
        emu.index_select = select
    for t in range(16):
        want = sorted(x for x in kept["hf"][0, t].tolist() if 0 <= x <= t)
        got = [x for x in kept["device"][t].tolist() if x >= 0]
        assert got == want, (t, got, want)
