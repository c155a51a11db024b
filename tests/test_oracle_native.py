"""The evaluator's native inner loops against the NumPy definitions they replace: contractions over packed weights
decoded inside the product, both scan recurrences (with either decay form), rank-to-ids; a quantised model through the
compiled graph with and without them."""
import numpy as np
import pytest

from poot_b200.oracle import native
from poot_b200.oracle.eval import EvalOptions, _matmul, _scan, eval_graph
from poot_b200.quant import codec
from poot_b200.tensor import DType


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0", "Q6_K", "Q5_0", "MXFP4", "Q2_K", "BF16", "F16"])
@pytest.mark.parametrize("narrow", [False, True])
def test_packed_matmul_equals_dequantise_then_multiply(fmt, narrow):
    rng = np.random.default_rng(0)
    N, K, M = 37, 512, 5
    w = (rng.standard_normal((N, K)) * 0.1).astype(np.float32)
    packed = codec.quantize(fmt, w) if fmt not in ("BF16",) else (w.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(-1)
    deq = codec.dequantize(fmt, packed, (N, K))
    x = rng.standard_normal((2, M, K)).astype(np.float32)
    want = _matmul(x.reshape(-1, K), deq.T, "narrow" if narrow else "exact", DType.BF16).reshape(2, M, N)
    got = native.packed_matmul(x, packed, fmt, (N, K), narrow)
    assert got.shape == (2, M, N) and np.abs(got - want).max() <= 2e-5 * np.abs(want).max() + 1e-6     # summation order only
    assert np.array_equal(got, native.packed_matmul(x, packed, fmt, (N, K), narrow, threads=1))        # thread count changes nothing


@pytest.mark.parametrize("per_channel", [False, True])
def test_scans_equal_the_token_loops(per_channel):
    rng = np.random.default_rng(1)
    H, L, D = 3, 9, 8
    r = lambda *s: rng.standard_normal(s).astype(np.float32)
    ins = [r(1, H, L, D), r(1, H, L, D), r(1, H, L, D), -np.abs(r(1, H, L, D if per_channel else 1)), np.abs(r(1, H, L, 1)) * 0.5,
           r(1, H, D, D) * 0.1]
    assert np.allclose(native.scan("delta_rule", ins), _scan("delta_rule", ins), atol=2e-5)
    N, P = 4, 6
    ssd = [r(1, H, L, P), r(1, H, L, N), r(1, H, L, N), np.abs(r(1, H, L, 1)) * 0.3, -np.abs(r(1, H, 1, 1)), r(1, H, 1, 1), r(1, H, N, P) * 0.1]
    assert np.allclose(native.scan("ssd", ssd), _scan("ssd", ssd), atol=2e-5)


def test_arg_top_k_places_every_ranked_entry():
    rank = np.array([[2, 0, 5, 1, 3], [4, 3, 2, 1, 0], [9, 9, 0, 9, 9]], np.int32)
    assert native.arg_top_k(rank, 3).tolist() == [[1, 3, 0], [4, 3, 2], [2, 0, 0]]


def test_packed_graph_through_the_compiler_natively():
    """A gated FFN stack over packed weights: the compiled graph (packed contractions formed) evaluated with the native
    loops equals the NumPy evaluation of the same graph to summation order, with no f32 copy of any matrix."""
    from poot_b200.ir import oplib as O
    from poot_b200.ir.builder import Builder
    from poot_b200.plan import compile_graph
    from poot_b200.quant.formats import packed_nbytes
    H, F, L = 256, 512, 7
    rng = np.random.default_rng(3)
    b = Builder()
    x = b.slot("x", (L, H), DType.F32, "activation")
    feed = {"x": rng.standard_normal((L, H)).astype(np.float32)}
    h = x
    for l, fmt in enumerate(("Q4_K", "Q8_0", "Q6_K")):
        ws = {}
        for role, (n, k) in (("gate", (F, H)), ("up", (F, H)), ("down", (H, F))):
            name = f"l{l}.{role}"
            feed[name] = codec.quantize(fmt, (rng.standard_normal((n, k)) * 0.05).astype(np.float32))
            raw = b.const(name, (packed_nbytes(fmt, n * k),), DType.U8)
            ws[role] = b.packed_dequant(raw, fmt, (n, k))
        h = h + O.linear(b, O.swiglu(b, O.linear(b, h, ws["gate"]), O.linear(b, h, ws["up"])), ws["down"])
    b.output(h, "out", "result")
    prog = compile_graph(b.finish())
    def count(g):                  # some contractions sit inside an epilogue composite's body
        return sum((e.op == "packed_contraction") + (count(e.body) if e.body is not None and e.op != "packed_contraction" else 0) for e in g.eqns)
    assert count(prog.graph) == 9
    want = eval_graph(prog.graph, feed, EvalOptions(matmul_precision="exact")).outputs["out"]
    got = eval_graph(prog.graph, feed, EvalOptions(matmul_precision="exact", native=True)).outputs["out"]
    assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    # under narrow operands a sum that differs in its last bit may round an activation the other way: one bf16 step
    narrow = eval_graph(prog.graph, feed).outputs["out"]
    assert np.abs(eval_graph(prog.graph, feed, EvalOptions(native=True)).outputs["out"] - narrow).max() <= 1e-2 * np.abs(narrow).max()


def test_quantised_gguf_is_served_by_the_oracle_at_its_packed_size(tmp_path):
    """A Q4_K / Q8_0 GGUF through ``LLM.oracle(packed=True)``: the matrices stay as stored bytes (no f32 copies), the
    step graphs declare them packed, and the greedy continuation equals the oracle over the decoded weights."""
    import dataclasses
    from poot_b200.driver.handle import ModelHandle, write_random_gguf
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.llm import LLM
    from poot_b200.models.config import tiny_llama
    cfg = dataclasses.replace(tiny_llama(), ffn=768, vocab=4096, bos_token=1, eos_token=2)
    path = str(tmp_path / "tiny-q4k.gguf")
    write_random_gguf(path, cfg, "Q4_K", "Q8_0", seed=0, std=0.05)
    weights, formats = ModelHandle.load(path).packed_oracle_weights()
    assert formats["layers.0.attn_q"] == "Q4_K" and formats["embed"] == "Q8_0" and weights["layers.0.attn_q"].dtype == np.uint8
    dense_bytes = sum(v.nbytes for v in ModelHandle.load(path).oracle_weights().values())
    assert sum(v.nbytes for v in weights.values()) < 0.3 * dense_bytes
    prompt = [int(t) for t in np.random.default_rng(4).integers(3, 4096, 21)]
    p = SamplingParams(max_tokens=6, ignore_eos=True)
    want = LLM.oracle(path, rows=1, max_seq=64, num_blocks=8, prefill_chunk=16).generate_tokens(prompt, p)
    packed = LLM.oracle(path, rows=1, max_seq=64, num_blocks=8, prefill_chunk=16, packed=True)
    assert packed.generate_tokens(prompt, p) == want
    graphs = list(packed.driver.engine.inner.graphs.values())
    assert graphs and all(any(e.op == "packed_contraction" for e in gr.eqns) and any(e.op == "packed_row_gather" for e in gr.eqns) for gr in graphs)
