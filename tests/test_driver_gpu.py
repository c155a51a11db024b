"""The serving driver and the public ``LLM`` API on the device engine.

Generated tokens are checked against the fp32 PyTorch restatement of the stack by teacher forcing: the reference
logits of the full (prompt + generated) sequence must rank every generated token first, up to a near-tie margin
(bf16 kernels may legitimately flip picks whose reference logits are closer than the margin).
"""
import json
import http.client

import pytest
import torch

pytestmark = pytest.mark.gpu

TIE = 0.08


def _llm(**kw):
    from poot_b200.llm import LLM
    args = dict(rows=4, max_seq=256, prefill_chunk=64, num_blocks=96, std=0.05, vocab=4096)
    args.update(kw)
    return LLM.random("tiny-llama", **args)


def _check_greedy(llm, prompt, gen):
    from poot_b200.oracle.torch_ref import forward_logits
    seq = torch.tensor(list(prompt) + list(gen), dtype=torch.int32, device="cuda")
    ref = forward_logits(llm.engine.w, seq)
    for i, tok in enumerate(gen):
        row = ref[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - TIE, (i, tok, int(row.argmax()), float(row.max() - row[tok]))


def _prompt(n, seed, vocab=4096):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(3, vocab, (n,), generator=g).tolist()


def test_generate_with_chunked_prefill_matches_reference():
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.ops import cuda_ops as K
    llm = _llm()
    prompt = _prompt(150, 0)                   # 150 tokens > chunk 64: three prefill pieces
    gen = llm.generate_tokens(prompt, SamplingParams(max_tokens=12, ignore_eos=True))
    K.check_status()
    assert len(gen) == 12
    _check_greedy(llm, prompt, gen)
    assert llm.driver.stats["prefill_tokens"] >= 150 and llm.driver.kv_usage()["blocks_used"] <= 9  # only cached prefix blocks stay


def test_continuous_batching_mixed_prefill_and_decode():
    from poot_b200.driver.sampler import SamplingParams
    llm = _llm()
    d = llm.driver
    prompts = [_prompt(n, s) for n, s in ((20, 1), (90, 2), (5, 3))]
    gens = {}
    sids = [d.open(prompts[0], SamplingParams(max_tokens=10, ignore_eos=True))]
    live = {sids[0]: 0}
    step = 0
    while live:
        if step == 2:                          # two late arrivals join while the first sequence decodes
            for i in (1, 2):
                sid = d.open(prompts[i], SamplingParams(max_tokens=10, ignore_eos=True))
                live[sid] = i
        for r in d.step(list(live)):
            if r.token is None:
                continue
            d.commit(r.seq_id, [r.token])
            gens.setdefault(live[r.seq_id], []).append(r.token)
            if d.finished(r.seq_id, r.token):
                d.release(r.seq_id)
                del live[r.seq_id]
        step += 1
        assert step < 100
    for i in range(3):
        assert len(gens[i]) == 10
        _check_greedy(llm, prompts[i], gens[i])
    assert d.kv_usage()["blocks_used"] == d.kv_usage()["prefix_entries"]


def test_prefix_cache_hit_reuses_blocks_and_keeps_the_answer():
    from poot_b200.driver.sampler import SamplingParams
    llm = _llm()
    prompt = _prompt(70, 4)
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a = llm.generate_tokens(prompt, sp)
    hit0 = llm.driver.stats["prefix_hit_tokens"]
    b = llm.generate_tokens(prompt, SamplingParams(max_tokens=6, ignore_eos=True))
    assert llm.driver.stats["prefix_hit_tokens"] - hit0 == 64        # four full blocks of the 70-token prompt
    _check_greedy(llm, prompt, a)
    _check_greedy(llm, prompt, b)


def test_seeded_sampling_is_reproducible_and_bias_wins():
    from poot_b200.driver.sampler import SamplingParams
    llm = _llm()
    prompt = _prompt(16, 5)
    sp = dict(temperature=0.9, top_k=50, top_p=0.9, seed=1234, max_tokens=10, ignore_eos=True)
    a = llm.generate_tokens(prompt, SamplingParams(**sp))
    b = llm.generate_tokens(prompt, SamplingParams(**sp))
    c = llm.generate_tokens(prompt, SamplingParams(**{**sp, "seed": 99}))
    assert a == b and a != c
    forced = llm.generate_tokens(prompt, SamplingParams(max_tokens=5, ignore_eos=True, logit_bias={7: 100.0}))
    assert forced == [7] * 5
    lp = SamplingParams(max_tokens=4, ignore_eos=True, logprobs=1)
    d = llm.driver
    sid = d.open(prompt, lp)
    got = []
    while len(got) < 4:
        for r in d.step([sid]):
            if r.token is not None:
                d.commit(sid, [r.token])
                got.append(r.logprob)
    d.release(sid)
    assert all(x is not None and -20.0 < x <= 0.0 for x in got)


def test_guided_choice_on_device():
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.text.guided import build_constraint
    llm = _llm()
    d = llm.driver
    g = build_constraint({"choice": ["yes", "no", "maybe"]}, llm.tokenizer, d.eos_token)
    sid = d.open(llm.tokenizer.encode("answer:"), SamplingParams(max_tokens=16), guided=g)
    out = []
    for _ in range(16):
        r = d.step([sid])[0]
        d.commit(sid, [r.token])
        if d.finished(sid, r.token):
            if r.token != d.eos_token:
                out.append(r.token)
            break
        out.append(r.token)
    d.release(sid)
    assert llm.tokenizer.decode(out) in ("yes", "no", "maybe")


def test_http_server_over_the_device_engine():
    from poot_b200.serve import Metrics, ServeConfig, ServeEngine, Server, ServerState
    llm = _llm()
    cfg = ServeConfig(model="random:tiny-llama", addr="127.0.0.1:0", rows=4)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics())
    srv = Server(ServerState(eng, cfg, "tiny"))
    eng.start()
    srv.start()
    try:
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=120)
        c.request("POST", "/v1/completions", json.dumps({"prompt": _prompt(40, 6), "max_tokens": 8, "temperature": 0,
                                                         "ignore_eos": True}), {"Content-Type": "application/json"})
        r = c.getresponse()
        body = json.loads(r.read())
        assert r.status == 200, body
        assert body["usage"]["completion_tokens"] == 8 and body["choices"][0]["finish_reason"] == "length"
        c.request("GET", "/health")
        assert c.getresponse().read() and eng.health()["status"] == "serving"
    finally:
        srv.shutdown()


def test_quantised_gguf_checkpoint_end_to_end(tmp_path):
    """Q4_K projections + Q8_0 embeddings written to a GGUF file, loaded packed, decoded with the fused GEMV."""
    import dataclasses
    from poot_b200.driver.handle import ModelHandle, device_weights, write_random_gguf
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.llm import LLM
    from poot_b200.models.config import tiny_llama
    from poot_b200.ops import cuda_ops as K
    from poot_b200.oracle.torch_ref import forward_logits
    cfg = dataclasses.replace(tiny_llama(), ffn=768, vocab=4096, bos_token=1, eos_token=2)
    path = str(tmp_path / "tiny-q4k.gguf")
    write_random_gguf(path, cfg, "Q4_K", "Q8_0", seed=0, std=0.05)
    llm = LLM.load(path, rows=2, max_seq=128, prefill_chunk=32, num_blocks=32)
    assert isinstance(llm.engine.w.layers[0].wqkv, K.QuantWeight)
    prompt = _prompt(24, 7)
    gen = llm.generate_tokens(prompt, SamplingParams(max_tokens=8, ignore_eos=True))
    K.check_status()
    dense = device_weights(ModelHandle.load(path), "cuda", keep_packed=False)
    seq = torch.tensor(prompt + gen, dtype=torch.int32, device="cuda")
    ref = forward_logits(dense, seq)
    for i, tok in enumerate(gen):
        row = ref[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - TIE, (i, tok, int(row.argmax()))
