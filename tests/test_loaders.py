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
