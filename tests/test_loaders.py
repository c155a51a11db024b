"""GGUF and safetensors: round trips, zero-copy packed payloads, hostile inputs, name tables."""
import json
import struct

import numpy as np
import pytest

from poot_b200.load import gguf, names, safetensors as st
from poot_b200.quant import codec
from poot_b200.quant.formats import UnsupportedFormat
from poot_b200.quant.weights import PackedWeight
from poot_b200.tensor import DType


def _gguf(tmp_path, tensors, meta=None):
    p = str(tmp_path / "m.gguf")
    gguf.write_gguf(p, meta or {"general.architecture": "llama", "llama.block_count": 2}, tensors)
    return p


def test_gguf_round_trip_with_quantised_tensors(tmp_path):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((16, 512)) * 0.02).astype(np.float32)
    ts = [PackedWeight("blk.0.attn_q.weight", "Q4_K", w.shape, codec.quantize("Q4_K", w)),
          PackedWeight("token_embd.weight", "Q8_0", w.shape, codec.quantize("Q8_0", w)),
          PackedWeight("output_norm.weight", "F32", (512,), np.ones(512, dtype=np.float32).view(np.uint8))]
    store = gguf.read_gguf(_gguf(tmp_path, ts, {"general.architecture": "llama", "llama.block_count": 2,
                                                "tokenizer.ggml.tokens": ["a", "b"], "llama.rope.freq_base": 500000.0}))
    assert store.metadata["general.architecture"] == "llama" and store.metadata["tokenizer.ggml.tokens"] == ["a", "b"]
    assert store["blk.0.attn_q.weight"].format == "Q4_K" and store["blk.0.attn_q.weight"].shape == (16, 512)
    assert np.array_equal(store["blk.0.attn_q.weight"].to_f32(), codec.dequantize("Q4_K", ts[0].payload, w.shape))
    assert np.array_equal(store["output_norm.weight"].to_f32(), np.ones(512, dtype=np.float32))


def test_gguf_expert_stack_becomes_one_owner_per_expert(tmp_path):
    w = (np.random.default_rng(1).standard_normal((4, 8, 256)) * 0.02).astype(np.float32)
    t = PackedWeight("blk.0.ffn_gate_exps.weight", "Q8_0", w.shape, codec.quantize("Q8_0", w))
    store = gguf.read_gguf(_gguf(tmp_path, [t]))
    assert sorted(store.names()) == [f"blk.0.ffn_gate_exps.weight#{e}" for e in range(4)]
    assert np.allclose(store["blk.0.ffn_gate_exps.weight#2"].to_f32(), w[2], atol=1e-3)
    assert names.canonical_from_gguf("blk.0.ffn_gate_exps.weight#2") == "layers.0.experts.2.gate"


@pytest.mark.parametrize("mutate", ["magic", "truncate", "version", "huge_count"])
def test_gguf_hostile_headers_are_refused(tmp_path, mutate):
    p = _gguf(tmp_path, [PackedWeight("a", "F32", (4,), np.zeros(4, dtype=np.float32).view(np.uint8))])
    raw = bytearray(open(p, "rb").read())
    if mutate == "magic":
        raw[0] = 0
    elif mutate == "truncate":
        raw = raw[:30]
    elif mutate == "version":
        raw[4:8] = struct.pack("<I", 99)
    else:
        raw[8:16] = struct.pack("<Q", 1 << 40)
    open(p, "wb").write(raw)
    with pytest.raises(gguf.GgufError):
        gguf.read_gguf(p)


def test_gguf_refused_types_are_named(tmp_path):
    p = _gguf(tmp_path, [PackedWeight("a", "F32", (256,), np.zeros(256, dtype=np.float32).view(np.uint8))])
    raw = bytearray(open(p, "rb").read())
    # tensor directory entry: name (len 1, "a"), n_dims 1, dim 256, then the ggml type:
    # patch it to Q8_K (15), which exists in ggml but is refused by name
    entry = struct.pack("<Q", 1) + b"a" + struct.pack("<I", 1) + struct.pack("<Q", 256)
    pos = raw.find(entry) + len(entry)
    raw[pos:pos + 4] = struct.pack("<I", 15)
    open(p, "wb").write(raw)
    with pytest.raises(UnsupportedFormat, match="Q8_K"):
        gguf.read_gguf(p)


def test_safetensors_round_trip_and_hostile_inputs(tmp_path):
    p = str(tmp_path / "m.safetensors")
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.arange(8, dtype=np.uint16)
    st.write_safetensors(p, {"a": (DType.F32, a), "b": (DType.BF16, b)}, {"format": "pt"})
    ts = st.read_tensors(p)
    assert np.array_equal(st.as_numpy(*ts["a"]), a) and ts["b"][0] == DType.BF16
    store = st.load_weight_store(p)
    assert np.array_equal(store["a"].to_f32(), a)
    raw = open(p, "rb").read()
    (n,) = struct.unpack_from("<Q", raw, 0)
    header = json.loads(raw[8:8 + n])
    # duplicate key
    dup = raw[8:8 + n].decode().rstrip()[:-1] + ',"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    bad = str(tmp_path / "dup.safetensors")
    open(bad, "wb").write(struct.pack("<Q", len(dup)) + dup.encode() + raw[8 + n:])
    with pytest.raises(st.SafetensorsError, match="duplicate"):
        st.read_tensors(bad)
    # offsets that disagree with dtype x shape
    header["a"]["data_offsets"] = [0, 44]
    hj = json.dumps(header).encode()
    open(bad, "wb").write(struct.pack("<Q", len(hj)) + hj + raw[8 + n:])
    with pytest.raises(st.SafetensorsError):
        st.read_tensors(bad)
    # header length beyond the file
    open(bad, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(st.SafetensorsError):
        st.read_tensors(bad)


def test_name_tables_and_qk_permutation():
    assert names.canonical_from_hf("model.layers.3.self_attn.q_proj.weight") == "layers.3.attn_q"
    assert names.canonical_from_hf("model.layers.0.block_sparse_moe.experts.5.w3.weight") == "layers.0.experts.5.up"
    assert names.canonical_from_gguf("blk.7.attn_output.weight") == "layers.7.attn_o"
    assert names.canonical_from_hf("rotary.inv_freq") is None
    rows, heads = 64, 4
    fwd, inv = names.hf_to_gguf_qk_row_order(rows, heads), names.gguf_qk_row_order(rows, heads)
    w = np.arange(rows)
    assert np.array_equal(w[fwd][inv], w)


def test_lora_adapter_loads_merges_and_refuses(tmp_path):
    import json
    import numpy as np
    from poot_b200.load import lora
    from poot_b200.load.safetensors import write_safetensors
    from poot_b200.tensor import DType
    rng = np.random.default_rng(0)
    a = rng.standard_normal((4, 32)).astype(np.float32)
    b = rng.standard_normal((48, 4)).astype(np.float32)
    d = tmp_path / "adapter"
    d.mkdir()
    (d / "adapter_config.json").write_text(json.dumps({"peft_type": "LORA", "r": 4, "lora_alpha": 8}))
    write_safetensors(str(d / "adapter_model.safetensors"), {
        "base_model.model.model.layers.1.self_attn.q_proj.lora_A.weight": (DType.F32, a),
        "base_model.model.model.layers.1.self_attn.q_proj.lora_B.weight": (DType.F32, b)})
    ad = lora.load_adapter(str(d))
    assert ad.rank == 4 and ad.scale == 2.0 and list(ad.deltas) == ["layers.1.attn_q"]
    w = rng.standard_normal((48, 32)).astype(np.float32)
    merged = lora.merge_into({"layers.1.attn_q": w, "layers.1.attn_k": w}, ad)
    assert np.allclose(merged["layers.1.attn_q"], w + 2.0 * b @ a, atol=1e-5) and merged["layers.1.attn_k"] is w
    with pytest.raises(lora.LoraError):
        lora.merge_into({"layers.0.attn_q": w}, ad)
    with pytest.raises(lora.LoraError):
        lora.merge_into({"layers.1.attn_q": w[:, :16]}, ad)
    (d / "adapter_config.json").write_text(json.dumps({"peft_type": "LORA", "r": 4, "use_dora": True}))
    with pytest.raises(lora.LoraError):
        lora.load_adapter(str(d))
    (d / "adapter_config.json").write_text(json.dumps({"peft_type": "LORA", "r": 8}))
    with pytest.raises(lora.LoraError):
        lora.load_adapter(str(d))


def _write_tiny_hf(dirpath, seed=0):
    """A 2-layer Llama checkpoint in Hugging Face layout (config.json + model.safetensors)."""
    import json
    import numpy as np
    from poot_b200.load.safetensors import write_safetensors
    from poot_b200.tensor import DType
    cfg = {"model_type": "llama", "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
           "num_key_value_heads": 2, "intermediate_size": 96, "vocab_size": 300, "rms_norm_eps": 1e-5,
           "rope_theta": 10000.0, "max_position_embeddings": 128, "tie_word_embeddings": False, "head_dim": 16}
    (dirpath / "config.json").write_text(json.dumps(cfg))
    rng = np.random.default_rng(seed)

    def w(*shape):
        return (DType.F32, (rng.standard_normal(shape) * 0.1).astype(np.float32))
    t = {"model.embed_tokens.weight": w(300, 64), "model.norm.weight": (DType.F32, np.ones(64, np.float32)),
         "lm_head.weight": w(300, 64)}
    for l in range(2):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"] = (DType.F32, np.ones(64, np.float32))
        t[p + "post_attention_layernorm.weight"] = (DType.F32, np.ones(64, np.float32))
        t[p + "self_attn.q_proj.weight"] = w(64, 64)
        t[p + "self_attn.k_proj.weight"] = w(32, 64)
        t[p + "self_attn.v_proj.weight"] = w(32, 64)
        t[p + "self_attn.o_proj.weight"] = w(64, 64)
        t[p + "mlp.gate_proj.weight"] = w(96, 64)
        t[p + "mlp.up_proj.weight"] = w(96, 64)
        t[p + "mlp.down_proj.weight"] = w(64, 96)
    write_safetensors(str(dirpath / "model.safetensors"), t)
    return cfg


def test_model_handle_loads_hf_directory_and_merges_an_adapter(tmp_path):
    import json
    import numpy as np
    from poot_b200.driver.handle import ModelHandle
    from poot_b200.load import lora
    from poot_b200.load.safetensors import write_safetensors
    from poot_b200.oracle.runner import OracleSession
    from poot_b200.tensor import DType
    from poot_b200.weights import WeightMap
    _write_tiny_hf(tmp_path)
    h = ModelHandle.load(str(tmp_path))
    assert h.kind == "hf" and h.cfg.n_layers == 2 and h.cfg.n_kv_heads == 2 and not h.cfg.tie_embeddings
    assert WeightMap(h.canonical).missing(h.cfg) == []
    base = OracleSession(h.model, h.oracle_weights(), capacity=32).step(np.array([[5, 9, 200]]))
    rng = np.random.default_rng(1)
    ad = tmp_path / "ad"
    ad.mkdir()
    (ad / "adapter_config.json").write_text(json.dumps({"r": 2, "lora_alpha": 4}))
    write_safetensors(str(ad / "adapter_model.safetensors"), {
        "base_model.model.model.layers.0.mlp.down_proj.lora_A.weight": (DType.F32, rng.standard_normal((2, 96)).astype(np.float32)),
        "base_model.model.model.layers.0.mlp.down_proj.lora_B.weight": (DType.F32, rng.standard_normal((64, 2)).astype(np.float32))})
    before = h.f32("layers.0.ffn_down").copy()
    adapter = lora.load_adapter(str(ad))
    h.apply_adapter(adapter)
    assert h.adapter == "ad" and np.allclose(h.f32("layers.0.ffn_down"), before + adapter.delta("layers.0.ffn_down"), atol=1e-5)
    tuned = OracleSession(h.model, h.oracle_weights(), capacity=32).step(np.array([[5, 9, 200]]))
    assert np.isfinite(tuned).all() and np.abs(tuned - base).max() > 1e-3     # the adapter changes the logits


def test_phi3_fused_projections_are_cut_into_roles(tmp_path):
    import json
    import numpy as np
    from poot_b200.driver.handle import ModelHandle
    from poot_b200.load.safetensors import write_safetensors
    from poot_b200.tensor import DType
    from poot_b200.weights import WeightMap
    cfg = {"model_type": "phi3", "hidden_size": 64, "num_hidden_layers": 1, "num_attention_heads": 4,
           "num_key_value_heads": 2, "intermediate_size": 96, "vocab_size": 100, "max_position_embeddings": 128}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    rng = np.random.default_rng(0)
    qkv = rng.standard_normal((64 + 2 * 32, 64)).astype(np.float32)
    gu = rng.standard_normal((192, 64)).astype(np.float32)
    one = (DType.F32, np.ones(64, np.float32))
    write_safetensors(str(tmp_path / "model.safetensors"), {
        "model.embed_tokens.weight": (DType.F32, rng.standard_normal((100, 64)).astype(np.float32)),
        "model.norm.weight": one, "lm_head.weight": (DType.F32, rng.standard_normal((100, 64)).astype(np.float32)),
        "model.layers.0.input_layernorm.weight": one, "model.layers.0.post_attention_layernorm.weight": one,
        "model.layers.0.self_attn.qkv_proj.weight": (DType.F32, qkv),
        "model.layers.0.self_attn.o_proj.weight": (DType.F32, rng.standard_normal((64, 64)).astype(np.float32)),
        "model.layers.0.mlp.gate_up_proj.weight": (DType.F32, gu),
        "model.layers.0.mlp.down_proj.weight": (DType.F32, rng.standard_normal((64, 96)).astype(np.float32))})
    h = ModelHandle.load(str(tmp_path))
    assert WeightMap(h.canonical).missing(h.cfg) == []
    assert np.array_equal(h.f32("layers.0.attn_q"), qkv[:64]) and np.array_equal(h.f32("layers.0.attn_v"), qkv[96:])
    assert np.array_equal(h.f32("layers.0.ffn_gate"), gu[:96]) and np.array_equal(h.f32("layers.0.ffn_up"), gu[96:])
