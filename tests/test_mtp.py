"""Multi-token-prediction drafting: the layer's graph against a plain restatement, and drafting through the driver
(greedy output unchanged, the layer's cache kept in step with the target's, drafts accepted when the layer is right)."""
import numpy as np
import pytest

from poot_b200.driver.features import Feature, Incompatible, Unavailable, check, require_mtp
from poot_b200.driver.sampler import SamplingParams
from poot_b200.llm import LLM
from poot_b200.models.config import DecoderConfig, mtp_config
from poot_b200.models.model import Model, StepSpec
from poot_b200.oracle.eval import EvalOptions, eval_graph
from poot_b200.oracle.runner import random_weights_f32


def _cfg(**kw):
    base = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=128, vocab=97, max_position=256,
                mtp_layers=1)
    base.update(kw)
    return DecoderConfig(**base)


def _rms(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def test_mtp_config_is_one_block_of_the_kind_that_follows_the_stack():
    dense = mtp_config(_cfg())
    assert dense.n_layers == 1 and dense.mtp_head and not dense.moe_layer(0) and dense.mtp_layers == 0
    moe = mtp_config(_cfg(n_experts=4, top_k=2, moe_ffn=32, first_dense_layers=1))
    assert moe.moe_layer(0)                       # the layer after a routed stack is routed
    shapes = Model(dense).weight_shapes()
    assert shapes["mtp.eh_proj"] == (64, 128) and shapes["mtp.enorm"] == (64,) and "layers.1.attn_q" not in shapes
    with pytest.raises(ValueError):
        mtp_config(_cfg(mtp_layers=0))


def test_mtp_input_mix_matches_the_plain_statement():
    """One position, empty cache: attention over a single key is the value itself, so the whole layer can be restated
    in a few lines (a window of one key keeps that true away from position 0); position 0 zeroes the embedding, any
    other position keeps it."""
    cfg = mtp_config(_cfg(sliding_window=1))
    m = Model(cfg)
    w = random_weights_f32(m, seed=3, std=0.2)
    rng = np.random.default_rng(0)
    w["mtp.enorm"], w["mtp.hnorm"] = rng.uniform(0.5, 1.5, 64).astype(np.float32), rng.uniform(0.5, 1.5, 64).astype(np.float32)
    g = m.trace(StepSpec(rows=1, tokens=1, capacity=16, paged=True, pool_slots=32, logit_rows="all"))
    carry = rng.standard_normal((1, 64)).astype(np.float32)
    for pos in (0, 5):
        ins = {i.name: w[i.name] for i in g.inputs if i.storage == "const"}
        for i in g.inputs:
            if i.storage == "state":
                ins[i.name] = np.zeros(g.types[i.value].shape, np.float32)
        read = np.full((1, 16), 31, np.int32)
        read[0, pos] = 7
        ins.update(tokens=np.array([[11]], np.int32), positions=np.array([[pos]], np.int32), read_map=read,
                   write_map=np.array([7], np.int32), carry=carry)
        out = eval_graph(g, ins, EvalOptions(matmul_precision="exact")).outputs
        e = w["embed"][11] * (0.0 if pos == 0 else 1.0)
        h = np.concatenate([_rms(e, w["mtp.enorm"], cfg.norm_eps), _rms(carry[0], w["mtp.hnorm"], cfg.norm_eps)]) @ w["mtp.eh_proj"].T
        x = _rms(h, w["layers.0.attn_norm"], cfg.norm_eps)
        v = (w["layers.0.attn_v"] @ x).reshape(2, 16)
        h = h + w["layers.0.attn_o"] @ np.repeat(v, 2, axis=0).reshape(-1)          # softmax over one key = 1
        x = _rms(h, w["layers.0.ffn_norm"], cfg.norm_eps)
        gate, up = w["layers.0.ffn_gate"] @ x, w["layers.0.ffn_up"] @ x
        h = h + w["layers.0.ffn_down"] @ (gate / (1 + np.exp(-gate)) * up)
        hid = _rms(h, w["final_norm"], cfg.norm_eps)
        np.testing.assert_allclose(out["hidden"][0], hid, rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(out["logits"][0], w["lm_head"] @ hid, rtol=2e-4, atol=2e-5)


def _llm(k, mtp_seed=1, **kw):
    cfg = _cfg(**kw)
    target = Model(cfg)
    tw = random_weights_f32(target, seed=0, std=0.3)
    mw = random_weights_f32(Model(mtp_config(cfg)), seed=mtp_seed, std=0.3)
    mw["embed"], mw["lm_head"] = tw["embed"], tw["lm_head"]                     # the layer shares the target's tables
    plain = LLM.oracle_from(target, tw, rows=4, max_seq=128, num_blocks=64, prefill_chunk=16)
    drafted = LLM.oracle_from(target, tw, rows=4, max_seq=128, num_blocks=64, prefill_chunk=16, mtp=(mw, k))
    return plain, drafted


@pytest.mark.parametrize("k", [1, 3])
def test_drafting_with_the_layer_leaves_greedy_output_unchanged(k):
    plain, drafted = _llm(k)
    rng = np.random.default_rng(5)
    for n in (5, 23, 40):                       # one piece, two pieces (16 + 7), three
        prompt = rng.integers(3, 97, n).tolist()
        p = SamplingParams(max_tokens=12, ignore_eos=True)
        want = plain.generate_tokens(prompt, p)
        got = drafted.generate_tokens(prompt, p)
        assert got == want
    st = drafted.driver.stats
    assert st["draft_proposed"] > 0 and drafted.draft.stats["catch_up_steps"] > 0
    if k > 1:
        assert drafted.draft.stats["chain_steps"] > 0
    assert drafted.driver.prefix is None          # prefix reuse is off under this policy


def test_a_layer_that_knows_the_answer_has_its_drafts_accepted():
    """Stand-in for a trained layer: a runner that answers with the target's own greedy continuation.  Every draft is
    accepted, so a round of k drafts costs one target step for k + 1 tokens - and the cache bookkeeping (positions,
    slots, the tokens after each position) is checked on the way."""
    plain, drafted = _llm(3)
    prompt = list(range(10, 30))
    p = SamplingParams(max_tokens=16, ignore_eos=True)
    want = plain.generate_tokens(prompt, p)
    full = prompt + want
    real = drafted.draft.runner
    seen = []

    class Knowing:
        max_tokens = real.max_tokens
        block_tables = real.block_tables
        last_hidden = None

        def run_step(self, inp):
            T = inp.live_tokens
            seen.append((inp.positions[:T].copy(), inp.tokens[:T].copy(), inp.slots[:T].copy()))
            for pos, tok in zip(inp.positions[:T], inp.tokens[:T]):
                assert full[pos + 1] == tok or pos + 1 >= len(full), "the layer is fed the token after each position"
            picked = np.zeros((len(inp.logit_idx), 2), np.int32)
            for b in range(inp.live_rows):
                pos = int(inp.positions[inp.logit_idx[b]])
                picked[b, 0] = full[pos + 2] if pos + 2 < len(full) else 0
            picked[:, 1] = -1
            self.last_hidden = np.zeros((T, 64), np.float32)
            return picked, None

    drafted.draft.runner = Knowing()
    got = drafted.generate_tokens(prompt, p)
    assert got == want
    st = drafted.driver.stats
    assert st["draft_accepted"] == st["draft_proposed"] > 0
    assert st["steps"] < plain.driver.stats["steps"]            # fewer target steps for the same tokens
    # catch-up after the prompt covers every prompt position, at the slots the target used
    pos0, _, slots0 = seen[0]
    assert pos0.tolist() == list(range(len(pos0))) and (slots0 >= 0).all()


def test_mtp_feature_rules():
    require_mtp(_cfg())
    with pytest.raises(Unavailable):
        require_mtp(_cfg(mtp_layers=0))
    check([Feature.DRAFT_MTP])
    for other in (Feature.PREFIX_CACHE, Feature.BEAM, Feature.ADAPTERS, Feature.TENSOR_PLACEMENT, Feature.DRAFT_LOOKUP,
                  Feature.GUIDED):
        with pytest.raises(Incompatible):
            check([Feature.DRAFT_MTP, other])
    plain_model = Model(_cfg(mtp_layers=0))
    with pytest.raises(Unavailable):
        LLM.oracle_from(plain_model, random_weights_f32(plain_model), mtp=({}, 2))


def test_checkpoint_with_a_stored_layer_drafts_through_the_public_loader(tmp_path):
    """A DeepSeek-V3 style directory whose safetensors also hold ``model.layers.<n_layers>.*`` (the block, ``enorm``,
    ``hnorm``, ``eh_proj``, ``shared_head.norm``): ``LLM.oracle(path, draft_mtp=k)`` finds the layer, drafts with it and
    generates what the plain load generates.  A directory without those tensors refuses the flag with a typed error."""
    import json
    import torch
    from safetensors.torch import load_file, save_file
    from tests.test_hf_parity import CASES, build
    m, vocab = build(CASES["deepseek3"])
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    with pytest.raises(Unavailable):
        LLM.oracle(str(tmp_path), rows=4, max_seq=64, num_blocks=32, prefill_chunk=16, draft_mtp=2)
    cfg_path = tmp_path / "config.json"
    hf = json.loads(cfg_path.read_text())
    n = hf["num_hidden_layers"]
    hf["num_nextn_predict_layers"] = 1
    cfg_path.write_text(json.dumps(hf))
    with pytest.raises(Unavailable):          # the header names a layer the files do not store
        LLM.oracle(str(tmp_path), rows=4, max_seq=64, num_blocks=32, prefill_chunk=16, draft_mtp=2)
    st_path = tmp_path / "model.safetensors"
    tensors = load_file(str(st_path))
    g = torch.Generator().manual_seed(9)
    last = f"model.layers.{n - 1}."
    for name in [k for k in tensors if k.startswith(last)]:
        t = tensors[name]
        fresh = t.clone() if "bias" in name and t.dtype != torch.float32 else t + 0.05 * torch.randn(t.shape, generator=g).to(t.dtype)
        tensors[f"model.layers.{n}." + name[len(last):]] = fresh
    H = hf["hidden_size"]
    tensors[f"model.layers.{n}.enorm.weight"] = 1 + 0.1 * torch.randn(H, generator=g)
    tensors[f"model.layers.{n}.hnorm.weight"] = 1 + 0.1 * torch.randn(H, generator=g)
    tensors[f"model.layers.{n}.eh_proj.weight"] = 0.3 * torch.randn(H, 2 * H, generator=g)
    tensors[f"model.layers.{n}.shared_head.norm.weight"] = 1 + 0.1 * torch.randn(H, generator=g)
    save_file(tensors, str(st_path), metadata={"format": "pt"})
    plain = LLM.oracle(str(tmp_path), rows=4, max_seq=64, num_blocks=32, prefill_chunk=16)
    drafted = LLM.oracle(str(tmp_path), rows=4, max_seq=64, num_blocks=32, prefill_chunk=16, draft_mtp=2)
    assert drafted.handle.has_mtp and drafted.draft is not None
    mw = drafted.handle.mtp_oracle_weights()
    assert mw["mtp.eh_proj"].shape == (H, 2 * H) and "layers.0.experts_in" in mw and "final_norm" in mw
    assert not any(k.startswith(f"layers.{n}.") for k in plain.handle.oracle_weights())
    prompt = torch.randint(3, vocab, (21,), generator=g).tolist()
    p = SamplingParams(max_tokens=8, ignore_eos=True)
    assert drafted.generate_tokens(prompt, p) == plain.generate_tokens(prompt, p)
    assert drafted.driver.stats["draft_proposed"] > 0 and drafted.draft.stats["chain_steps"] > 0


def test_device_program_of_the_layer_under_emulated_kernels(tmp_path):
    """The engine's kernel program for the layer (embedding gather, position-0 zeroing, the two input norms, the split
    projection, one block, closing norm over every row, head) against the f32 evaluation of the layer's graph, and
    drafting through the device step engines end to end, all on host restatements of the kernels."""
    import torch
    from poot_b200.driver.engines import DeviceStepEngine, OracleStepEngine
    from poot_b200.driver.driver import StepInputs
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.weights import from_named_tensors
    from poot_b200.utils.kernel_emulation import emulated_kernels
    cfg = mtp_config(_cfg(hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512))
    layer = Model(cfg)
    w = random_weights_f32(layer, seed=4, std=0.08)
    rng = np.random.default_rng(1)
    w["mtp.enorm"], w["mtp.hnorm"] = rng.uniform(0.5, 1.5, 128).astype(np.float32), rng.uniform(0.5, 1.5, 128).astype(np.float32)
    # through bf16 once, so both sides hold the same numbers
    w = {k: torch.from_numpy(v).to(torch.bfloat16).float().numpy() for k, v in w.items()}
    T = 6
    tokens = rng.integers(3, 512, T).astype(np.int32)
    carry = torch.from_numpy(rng.standard_normal((T, 128)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    pos = np.arange(T, dtype=np.int32)
    slots = (16 + pos).astype(np.int32)                     # block 1 of the pool
    params = np.zeros((1, 4), np.float32); params[:, 0] = 1.0; params[:, 1] = -1e30; params[:, 3] = 1.0
    mk = lambda: StepInputs(tokens, pos, slots, np.zeros(T, np.int32), pos + 1, np.array([T - 1], np.int64), 0, params,
                            np.zeros(1, np.int32), np.zeros(1, np.int32), None, False, T, 1, carry=carry)
    ref = OracleStepEngine(layer, w, num_blocks=4, max_seqs=2, max_tokens=16, max_blocks_per_seq=2)
    ref.write_block_table(0, [1])
    want_pick, _ = ref.run_step(mk())
    with emulated_kernels():
        dw = from_named_tensors(cfg, {k: torch.from_numpy(v) for k, v in w.items()}, "cpu")
        eng = DecoderEngine(dw, num_blocks=4, max_seqs=2, max_tokens=16, max_blocks_per_seq=2, device="cpu", use_graphs=False)
        assert eng.carry and eng.program is None
        dev = DeviceStepEngine(eng)
        dev.write_block_table(0, [1])
        got_pick, _ = dev.run_step(mk())
        hid = dev.last_hidden[:T]
        err = np.abs(hid - ref.last_hidden).max() / np.abs(ref.last_hidden).max()
        assert err < 0.03, err
        lg = np.abs(eng.logits[0].numpy() - ref.last_logits(1)[0]).max() / np.abs(ref.last_logits(1)[0]).max()
        assert lg < 0.03, lg
        assert int(got_pick[0, 0]) == int(want_pick[0, 0]) or lg < 0.03
        # end to end: random-init target + layer on the device step engines; greedy output is what plain decoding gives
        over = dict(n_layers=2, hidden=128, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512, max_position=256,
                    mtp_layers=1)
        plain = LLM.random("tiny-llama", device="cpu", rows=4, max_seq=128, prefill_chunk=16, num_blocks=64, std=0.08, **over)
        drafted = LLM.random("tiny-llama", device="cpu", rows=4, max_seq=128, prefill_chunk=16, num_blocks=64, std=0.08,
                             draft_mtp=3, **over)
        assert drafted.mtp_engine.block_tables is drafted.engine.block_tables
        assert drafted.mtp_engine.w.embed is drafted.engine.w.embed
        prompt = rng.integers(3, 512, 21).tolist()
        p = SamplingParams(max_tokens=10, ignore_eos=True)
        assert drafted.generate_tokens(prompt, p) == plain.generate_tokens(prompt, p)
        assert drafted.driver.stats["draft_proposed"] > 0 and drafted.draft.stats["chain_steps"] > 0
