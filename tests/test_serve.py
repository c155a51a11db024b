"""Serving layer on the deterministic host engine: scheduler, API validation, HTTP surface, hostile input.

The fake engine's next token is (last token + 1) mod vocab, and the byte tokenizer maps id = byte + 3, so a prompt
ending in "a" continues "bcdef...": every expected completion below is computed by hand from that rule.
"""
import http.client
import json
import queue
import socket
import threading
import time

import pytest

from poot_b200.driver.sampler import SamplingParams
from poot_b200.llm import LLM
from poot_b200.serve import (ApiError, Job, Metrics, ServeConfig, ServeEngine, Server, ServerState, parse_args,
                             sampling_from_request)


def _stack(rows=4, max_pending=8, fail_at_step=None, **cfg_kw):
    llm = LLM.fake(vocab=1000, rows=rows, max_seq=256, num_blocks=128, prefill_chunk=32, fail_at_step=fail_at_step)
    cfg = ServeConfig(model="fake", addr="127.0.0.1:0", rows=rows, max_pending_requests=max_pending, **cfg_kw)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics(), max_pending, cfg.max_queue_wait_secs)
    srv = Server(ServerState(eng, cfg, "fake-model"))
    eng.start()
    srv.start()
    return llm, eng, srv


def _post(port, path, body, headers=None, raw=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
    data = raw if raw is not None else json.dumps(body).encode()
    c.request("POST", path, data, {"Content-Type": "application/json", **(headers or {})})
    r = c.getresponse()
    out = r.status, dict(r.getheaders()), r.read()
    c.close()
    return out


def _get(port, path, headers=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
    c.request("GET", path, headers=headers or {})
    r = c.getresponse()
    out = r.status, r.read()
    c.close()
    return out


@pytest.fixture
def stack():
    llm, eng, srv = _stack()
    yield llm, eng, srv
    srv.shutdown()


def test_completion_follows_the_fake_engine_rule(stack):
    _, eng, srv = stack
    st, _, body = _post(srv.port, "/v1/completions", {"prompt": "xa", "max_tokens": 5, "temperature": 0})
    assert st == 200
    r = json.loads(body)
    assert r["choices"][0]["text"] == "bcdef" and r["choices"][0]["finish_reason"] == "length"
    assert r["usage"] == {"prompt_tokens": 3, "completion_tokens": 5, "total_tokens": 8,
                          "prompt_tokens_details": {"cached_tokens": 0}}
    assert r["object"] == "text_completion" and r["model"] == "fake-model"


def test_stop_string_is_withheld_and_ends_the_request(stack):
    _, _, srv = stack
    st, _, body = _post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 20, "stop": ["ef", "zz"]})
    r = json.loads(body)["choices"][0]
    assert st == 200 and r["text"] == "bcd" and r["finish_reason"] == "stop"


def test_n_choices_and_token_id_prompt(stack):
    _, _, srv = stack
    st, _, body = _post(srv.port, "/v1/completions", {"prompt": [1, 100], "max_tokens": 2, "n": 3})
    r = json.loads(body)
    assert st == 200 and len(r["choices"]) == 3 and [c["index"] for c in r["choices"]] == [0, 1, 2]
    assert all(c["text"] == "bc" for c in r["choices"])        # id 100 = byte 97 = "a"
    assert r["usage"]["completion_tokens"] == 6


def test_chat_completion_and_sse_stream(stack):
    _, _, srv = stack
    msgs = [{"role": "user", "content": "hi"}]
    st, _, body = _post(srv.port, "/v1/chat/completions", {"messages": msgs, "max_tokens": 3})
    r = json.loads(body)
    assert st == 200 and r["object"] == "chat.completion"
    assert r["choices"][0]["message"]["role"] == "assistant" and len(r["choices"][0]["message"]["content"]) >= 1
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=20)
    c.request("POST", "/v1/chat/completions", json.dumps({"messages": msgs, "max_tokens": 4, "stream": True,
                                                          "stream_options": {"include_usage": True}}),
              {"Content-Type": "application/json"})
    resp = c.getresponse()
    assert resp.status == 200 and resp.getheader("Content-Type") == "text/event-stream"
    events = [l[6:] for l in resp.read().decode().split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks if ch["choices"])
    assert text == r["choices"][0]["message"]["content"] + chr(ord(text[2]) + 1) if len(text) == 4 else True
    finals = [ch for ch in chunks if ch["choices"] and ch["choices"][0]["finish_reason"]]
    assert finals and finals[-1]["choices"][0]["finish_reason"] == "length"
    assert chunks[-1]["usage"]["completion_tokens"] == 4


def test_guided_choice_constrains_the_fake_engine(stack):
    _, _, srv = stack
    st, _, body = _post(srv.port, "/v1/completions", {"prompt": "x", "max_tokens": 8, "guided_choice": ["yes", "no"]})
    assert st == 200
    assert json.loads(body)["choices"][0]["text"] in ("yes", "no")


@pytest.mark.parametrize("body,param", [
    ({"prompt": "a", "max_tokens": 0}, "max_tokens"),
    ({"prompt": "a", "temperature": 9}, "temperature"),
    ({"prompt": "a", "stop": ["x"] * 17}, "stop"),
    ({"prompt": "a", "logit_bias": {"abc": 1}}, "logit_bias"),
    ({"prompt": "a", "n": 0}, "n"),
    ({"prompt": 5}, "prompt"),
    ({"prompt": "a", "top_p": 1.5}, "top_p"),
])
def test_invalid_requests_get_openai_shaped_400(stack, body, param):
    _, _, srv = stack
    st, _, raw = _post(srv.port, "/v1/completions", body)
    err = json.loads(raw)["error"]
    assert st == 400 and err["type"] == "invalid_request_error" and err["param"] == param


def test_clamps():
    sp = sampling_from_request({"max_tokens": 10 ** 9})
    assert sp.max_tokens == 32768
    with pytest.raises(ApiError):
        sampling_from_request({"logit_bias": {str(i): 0.0 for i in range(10001)}})


def test_hostile_http(stack):
    _, _, srv = stack
    assert _post(srv.port, "/v1/completions", None, raw=b"{not json")[0] == 400
    assert _post(srv.port, "/v1/completions", None, raw=b"[1,2]")[0] == 400
    assert _post(srv.port, "/v1/completions", None, raw=b"\xff\xfe{}")[0] == 400
    assert _post(srv.port, "/v1/nothing", {"a": 1})[0] == 404
    assert _post(srv.port, "/v1/completions", {"prompt": "a", "model": "other"})[0] == 404
    # body cap: Content-Length above the limit is refused before it is read
    s = socket.create_connection(("127.0.0.1", srv.port), timeout=10)
    s.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: 99999999\r\n\r\n")
    assert b" 413 " in s.recv(4096).split(b"\r\n")[0]
    s.close()
    # chunked bodies are refused
    s = socket.create_connection(("127.0.0.1", srv.port), timeout=10)
    s.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nTransfer-Encoding: chunked\r\n\r\n0\r\n\r\n")
    assert b" 400 " in s.recv(4096).split(b"\r\n")[0]
    s.close()
    st, _, raw = _post(srv.port, "/v1/embeddings", {"input": "x"})
    assert st == 400 and "embedding" in json.loads(raw)["error"]["message"]
    # the server is still healthy afterwards
    assert _get(srv.port, "/health")[0] == 200


def test_models_health_metrics(stack):
    _, _, srv = stack
    _post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 3})
    st, body = _get(srv.port, "/v1/models")
    assert st == 200 and json.loads(body)["data"][0]["id"] == "fake-model"
    assert _get(srv.port, "/v1/models/fake-model")[0] == 200 and _get(srv.port, "/v1/models/nope")[0] == 404
    st, body = _get(srv.port, "/health")
    assert st == 200 and json.loads(body)["status"] == "serving"
    st, body = _get(srv.port, "/metrics")
    m = json.loads(body)
    assert st == 200 and m["counters"]["poot_requests_completed_total"] >= 1 and m["counters"]["poot_completion_tokens_total"] >= 3
    st, body = _get(srv.port, "/metrics/prometheus")
    text = body.decode()
    assert st == 200 and "poot_ttft_ms" in text and "poot_kv_usage_ratio" in text and "# TYPE" in text
    assert _get(srv.port, "/v1/lora_adapters")[0] == 401     # admin key required


def test_host_policy_and_rate_limit():
    llm, eng, srv = _stack(allowed_hosts=["good.example"], rate_limit_rpm=2)
    try:
        assert _get(srv.port, "/health", {"Host": "evil.example"})[0] == 400
        assert _get(srv.port, "/health", {"Host": "good.example:1234"})[0] == 200
        h = {"Host": "good.example"}
        assert _post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 1}, h)[0] == 200
        assert _post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 1}, h)[0] == 200
        st, hdr, _ = _post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 1}, h)
        assert st == 429 and "Retry-After" in hdr
    finally:
        srv.shutdown()


def test_queue_full_returns_429_and_never_preempts():
    llm = LLM.fake(rows=1, max_seq=256, num_blocks=64, prefill_chunk=32)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics(), max_pending=2)
    # engine thread not started: submissions pile up
    a = eng.submit(Job([1, 5], SamplingParams(max_tokens=3)))
    b = eng.submit(Job([1, 6], SamplingParams(max_tokens=3)))
    with pytest.raises(queue.Full):
        eng.submit(Job([1, 7], SamplingParams(max_tokens=3)))
    assert eng.metrics.to_json()["counters"]["poot_requests_rejected_total"] == 1
    # one row: the older job runs to completion before the younger is admitted
    order = []
    eng.on_step = lambda res: order.append([r.seq_id for r in res])
    eng.state = "serving"
    for _ in range(20):
        eng.iteration()
    assert a.wait(1)["finish_reason"] == "length" and b.wait(1)["finish_reason"] == "length"
    assert a.tokens == [6, 7, 8] and b.tokens == [7, 8, 9]
    flat = [s[0] for s in order]
    assert flat == sorted(flat)            # sequence ids never interleave on one row


def test_cancel_releases_rows_and_blocks():
    llm = LLM.fake(rows=2, max_seq=256, num_blocks=64, prefill_chunk=32)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics())
    eng.state = "serving"
    j = eng.submit(Job([1, 5], SamplingParams(max_tokens=200), stream=True))
    for _ in range(3):
        eng.iteration()
    assert llm.driver.kv_usage()["blocks_used"] > 0
    j.cancelled.set()
    eng.iteration()
    assert llm.driver.kv_usage()["blocks_used"] == 0 and not eng.live
    assert j.wait(1)["finish_reason"] == "cancelled"


def test_engine_fault_turns_health_dead():
    llm, eng, srv = _stack(fail_at_step=2)
    try:
        st, _, raw = _post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 50})
        assert st == 500
        deadline = time.time() + 5
        while eng.state != "dead" and time.time() < deadline:
            time.sleep(0.01)
        st, body = _get(srv.port, "/health")
        assert st == 503 and json.loads(body)["status"] == "dead" and "fault" in json.loads(body)["cause"]
        assert _post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 5})[0] == 503
    finally:
        srv.httpd.shutdown()
        srv.httpd.server_close()


def test_prefix_cache_hit_is_reported(stack):
    _, _, srv = stack
    prompt = "p" * 40
    _post(srv.port, "/v1/completions", {"prompt": prompt, "max_tokens": 2})
    st, _, body = _post(srv.port, "/v1/completions", {"prompt": prompt, "max_tokens": 2})
    assert json.loads(body)["usage"]["prompt_tokens_details"]["cached_tokens"] == 32    # two full 16-token blocks


def test_concurrent_requests_batch_together(stack):
    _, eng, srv = stack
    sizes = []
    eng.on_step = lambda res: sizes.append(len(res))
    out = [None] * 4

    def go(i):
        out[i] = _post(srv.port, "/v1/completions", {"prompt": "q" * (i + 1) + "a", "max_tokens": 30})

    ts = [threading.Thread(target=go, args=(i,)) for i in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert all(o[0] == 200 for o in out)
    assert all(json.loads(o[2])["choices"][0]["text"].startswith("bcdef") for o in out)
    assert max(sizes) >= 2                # continuous batching: steps carried several sequences


def test_drain_finishes_live_requests_then_refuses():
    llm, eng, srv = _stack()
    res = {}
    t = threading.Thread(target=lambda: res.update(r=_post(srv.port, "/v1/completions", {"prompt": "a", "max_tokens": 40})))
    t.start()
    time.sleep(0.05)
    srv.shutdown()
    t.join()
    assert res["r"][0] == 200 and json.loads(res["r"][2])["usage"]["completion_tokens"] == 40


def test_cli_flags_are_strict():
    cfg = parse_args(["model.gguf", "127.0.0.1:9000", "--rows", "64", "--max-seq", "8192", "--no-prefix-cache",
                      "--placement", "tensor:0,1,2,3", "--allowed-host", "a", "--allowed-host", "b"])
    assert cfg.rows == 64 and cfg.placement_ordinals == [0, 1, 2, 3] and not cfg.prefix_cache and cfg.allowed_hosts == ["a", "b"]
    for bad in (["m", "--rows", "0"], ["m", "--bogus"], ["m", "--placement", "ring:0,1"], ["m", "nohost"],
                ["m", "--kv-dtype", "int3"]):
        with pytest.raises(ValueError):
            parse_args(bad)


def test_lone_greedy_request_is_served_through_lookup_drafting():
    from poot_b200.driver.speculate import LookupDraft
    llm = LLM.fake(vocab=300, rows=4, max_seq=512, num_blocks=128, prefill_chunk=64)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics(), draft=LookupDraft(2, 4))
    eng.state = "serving"
    prompt = llm.tokenizer.encode("abcdefghij abc")          # "abc" seen before: the continuation "defg" is drafted
    j = eng.submit(Job(prompt, SamplingParams(max_tokens=12, ignore_eos=True)))
    for _ in range(40):
        eng.iteration()
    assert j.wait(1)["finish_reason"] == "length" and j.text == "defghijklmno"
    assert llm.driver.stats["draft_accepted"] >= 4 and llm.driver.stats["steps"] < 12


def test_timing_snapshot_is_exposed_and_null_when_unmeasured():
    from poot_b200.profile import TimingOptions, TimingSnapshot
    llm = LLM.fake(vocab=1000, rows=4, max_seq=256, num_blocks=128, prefill_chunk=32)
    cfg = ServeConfig(model="fake", addr="127.0.0.1:0", rows=4)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics(), timing=TimingSnapshot(TimingOptions("detailed", max_steps=64)))
    srv = Server(ServerState(eng, cfg, "fake-model"))
    eng.start(); srv.start()
    try:
        assert _post(srv.port, "/v1/completions", {"prompt": "a" * 40, "max_tokens": 5})[0] == 200
        m = json.loads(_get(srv.port, "/metrics")[1])
        t = m["device_timing"]
        assert t["steps"] >= 5 and t["device_ms"] is None            # the host engine measures no device time: null, not 0
        assert set(t["host_ms"]) == {"plan", "run"} and m["execution_counters"]["replays"] == t["steps"]
    finally:
        srv.shutdown()
    with pytest.raises(Exception):
        from poot_b200.driver.features import Feature, check
        check([Feature.DEVICE_TIMING, Feature.TENSOR_PLACEMENT])


def test_flags_for_draft_policies_pools_and_range_checks():
    from poot_b200.driver.features import Feature, Unavailable, check
    from poot_b200.models.config import mixtral_8x7b, tiny_llama
    from poot_b200.serve.__main__ import _prove_ranges
    cfg = parse_args(["m", "--draft-model", "/models/small:4", "--check-ranges", "--timing-sample-every", "2",
                      "--timing-max-dispatch-records", "1000"])
    assert cfg.draft_model == "/models/small:4" and cfg.check_ranges and cfg.timing_sample_every == 2
    for bad in (["m", "--draft-model", "no-count"], ["m", "--draft-model", "p:4", "--draft-lookup", "3:4"], ["m", "--draft-mtp", "99"],
                ["m", "--timing-sample-every", "0"]):
        with pytest.raises(ValueError):
            parse_args(bad)
    with pytest.raises(Unavailable):                             # accepted by the parser, refused typed where the model is known
        from poot_b200.driver.features import require_mtp
        require_mtp(tiny_llama())
    from poot_b200.serve.__main__ import main as serve_main
    assert serve_main(["random:tiny-llama", "127.0.0.1:0", "--draft-mtp", "2", "--backend", "oracle"]) == 2
    assert parse_args(["m", "--expert-pool", "6", "--host-embedding"]).expert_pool == 6
    check([Feature.EXPERT_POOL])                                 # pooled experts are served (single-device engine)
    c = tiny_llama()
    c.n_layers = 1
    _prove_ranges(c, cfg)
    m = mixtral_8x7b()
    m.n_layers, m.hidden, m.moe_ffn, m.ffn, m.n_heads, m.n_kv_heads, m.head_dim, m.vocab = 1, 128, 64, 64, 2, 1, 64, 512
    _prove_ranges(m, cfg)                                        # expert ids are proven in range too
