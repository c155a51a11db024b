"""OpenAI-compatible HTTP/1.1 server on the standard library (the reference server is std-only too).

Surface (website/docs/serve/api.md:33-76): ``POST /v1/completions``, ``POST /v1/chat/completions`` (JSON or SSE),
``POST /v1/embeddings`` and ``/v1/rerank`` (served when the model is an encoder checkpoint; refused otherwise),
``GET /v1/models[/{id}]``, ``/health``, ``/metrics``, ``/metrics/prometheus``, ``GET/POST/DELETE /v1/lora_adapters``
(admin key).  Hardening: 64 KiB header cap, body caps, Host policy, per-minute rate limit, bounded pending queue
(429 + Retry-After), request / write timeouts, clamps (``max_tokens`` <= 32768, <= 16 stop strings, <= 10 000
``logit_bias`` entries), OpenAI-shaped error bodies for the 400 / 408 / 413 / 429 / 500 / 503 classes.
"""
from __future__ import annotations

import hmac
import json
import queue
import socket
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional, Tuple

from ..driver.sampler import SamplingParams
from ..text import chat as chat_mod
from ..text import guided as guided_mod
from ..text import tools as tools_mod
from .config import ServeConfig
from .scheduler import EngineDead, Job, ServeEngine

MAX_HEADER_BYTES = 64 * 1024
MAX_TOKENS_CLAMP = 32768


class ApiError(Exception):
    def __init__(self, status: int, message: str, kind: str = "invalid_request_error", param: Optional[str] = None,
                 retry_after: Optional[int] = None):
        super().__init__(message)
        self.status, self.message, self.kind, self.param, self.retry_after = status, message, kind, param, retry_after

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": self.kind, "param": self.param, "code": None}}


def _num(d: dict, key: str, lo, hi, default, cast=float):
    v = d.get(key, default)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ApiError(400, f"{key} must be a number", param=key)
    v = cast(v)
    if not (lo <= v <= hi):
        raise ApiError(400, f"{key} must be in [{lo}, {hi}]", param=key)
    return v


def sampling_from_request(req: dict, default_max: int = 256) -> SamplingParams:
    stop = req.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    if not isinstance(stop, list) or len(stop) > 16 or not all(isinstance(s, str) and s for s in stop):
        raise ApiError(400, "stop must be a string or a list of at most 16 non-empty strings", param="stop")
    bias = req.get("logit_bias") or {}
    if not isinstance(bias, dict) or len(bias) > 10000:
        raise ApiError(400, "logit_bias must be an object with at most 10000 entries", param="logit_bias")
    try:
        bias = {int(k): float(v) for k, v in bias.items()}
    except (TypeError, ValueError):
        raise ApiError(400, "logit_bias keys must be token ids and values numbers", param="logit_bias") from None
    max_tokens = req.get("max_completion_tokens", req.get("max_tokens", default_max))
    if max_tokens is None:
        max_tokens = default_max
    if isinstance(max_tokens, bool) or not isinstance(max_tokens, int) or max_tokens < 1:
        raise ApiError(400, "max_tokens must be a positive integer", param="max_tokens")
    temp = _num(req, "temperature", 0.0, 2.0, 1.0)
    seed = req.get("seed")
    if seed is not None and (isinstance(seed, bool) or not isinstance(seed, int)):
        raise ApiError(400, "seed must be an integer", param="seed")
    lp = req.get("logprobs")
    return SamplingParams(
        temperature=temp, top_k=_num(req, "top_k", 0, 1 << 20, 40, int), top_p=_num(req, "top_p", 0.0, 1.0, 1.0 if temp == 0 else 0.95),
        min_p=_num(req, "min_p", 0.0, 1.0, 0.0 if temp == 0 else 0.05), repeat_penalty=_num(req, "repetition_penalty", 0.01, 10.0, 1.0),
        presence_penalty=_num(req, "presence_penalty", -2.0, 2.0, 0.0), frequency_penalty=_num(req, "frequency_penalty", -2.0, 2.0, 0.0),
        seed=seed, logit_bias=bias, max_tokens=min(max_tokens, MAX_TOKENS_CLAMP), stop=stop,
        ignore_eos=bool(req.get("ignore_eos", False)), logprobs=1 if lp else 0)


class RateLimiter:
    def __init__(self, rpm: int):
        self.rpm, self.hits, self.lock = rpm, [], threading.Lock()

    def allow(self) -> bool:
        if self.rpm <= 0:
            return True
        now = time.monotonic()
        with self.lock:
            self.hits = [t for t in self.hits if now - t < 60.0]
            if len(self.hits) >= self.rpm:
                return False
            self.hits.append(now)
            return True


class ServerState:
    def __init__(self, engine: ServeEngine, cfg: ServeConfig, model_id: str, family: str = "llama",
                 chat_template: Optional[str] = None, bos_text: str = "", eos_text: str = ""):
        self.engine, self.cfg, self.model_id, self.family = engine, cfg, model_id, family
        self.chat_template, self.bos_text, self.eos_text = chat_template, bos_text, eos_text
        self.limiter = RateLimiter(cfg.rate_limit_rpm)
        self.created = int(time.time())
        self.admin_key = None
        if cfg.lora_admin_key_file:
            with open(cfg.lora_admin_key_file) as f:
                self.admin_key = f.read().strip()
        self.adapters: Dict[str, dict] = {}
        self.embedder = getattr(engine, "embedder", None)    # set when the served model is an encoder
        self.vision = None                                   # vision front end (tower + preprocessing) of a served VLM


def make_handler(state: ServerState):
    eng, cfg = state.engine, state.cfg

    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "poot-b200"

        def log_message(self, fmt, *args):   # quiet by default
            pass

        def setup(self):
            super().setup()
            self.connection.settimeout(cfg.request_timeout_secs)

        # ---- plumbing ---------------------------------------------------------------------------------------
        def _send(self, status: int, body, ctype="application/json", extra: Optional[dict] = None):
            raw = body if isinstance(body, bytes) else json.dumps(body).encode()
            self.send_response(status)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(raw)))
            for k, v in (extra or {}).items():
                self.send_header(k, str(v))
            self.end_headers()
            self.wfile.write(raw)

        def _error(self, e: ApiError):
            extra = {"Retry-After": e.retry_after} if e.retry_after is not None else None
            self.close_connection = True     # the body may be unread: never reuse the connection after an error
            try:
                self._send(e.status, e.body(), extra=extra)
            except (BrokenPipeError, ConnectionResetError, socket.timeout):
                pass

        def _check_head(self):
            if sum(len(k) + len(v) + 4 for k, v in self.headers.items()) > MAX_HEADER_BYTES:
                raise ApiError(431, "request header too large")
            if cfg.allowed_hosts:
                host = (self.headers.get("Host") or "").split(":")[0]
                if host not in cfg.allowed_hosts:
                    raise ApiError(400, "Host not allowed")

        def _body(self) -> dict:
            te = self.headers.get("Transfer-Encoding")
            if te:
                raise ApiError(400, "chunked request bodies are not accepted")
            cl = self.headers.get("Content-Length")
            if cl is None or not cl.isdigit():
                raise ApiError(411, "Content-Length required")
            n = int(cl)
            if n > cfg.max_body_mib * 1024 * 1024:
                raise ApiError(413, f"request body exceeds {cfg.max_body_mib} MiB")
            try:
                raw = self.rfile.read(n)
            except socket.timeout:
                raise ApiError(408, "timed out reading the request body") from None
            if len(raw) != n:
                raise ApiError(400, "request body shorter than Content-Length")
            try:
                obj = json.loads(raw.decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as ex:
                raise ApiError(400, f"body is not valid JSON: {ex}") from None
            if not isinstance(obj, dict):
                raise ApiError(400, "body must be a JSON object")
            return obj

        # ---- routes -----------------------------------------------------------------------------------------
        def do_GET(self):
            try:
                self._check_head()
                path = self.path.split("?")[0]
                if path == "/health":
                    h = eng.health()
                    return self._send(200 if h["status"] == "serving" else 503, h)
                if path == "/metrics":
                    body = eng.metrics.to_json()
                    if eng.timing is not None:
                        from ..profile import Report
                        body["device_timing"] = Report.window(eng.timing, entries=256).to_json()
                        c = eng.timing.counters
                        body["execution_counters"] = {"dispatches": c.dispatches, "replays": c.replays}
                    return self._send(200, body)
                if path == "/metrics/prometheus":
                    return self._send(200, eng.metrics.to_prometheus().encode(), "text/plain; version=0.0.4")
                if path == "/v1/models":
                    return self._send(200, {"object": "list", "data": [self._model_obj()] + [
                        {"id": a["id"], "object": "model", "created": a["created"], "owned_by": "poot-b200", "parent": state.model_id}
                        for a in state.adapters.values()]})
                if path.startswith("/v1/models/"):
                    if path[len("/v1/models/"):] != state.model_id:
                        raise ApiError(404, "model not found", "not_found_error")
                    return self._send(200, self._model_obj())
                if path == "/v1/lora_adapters":
                    self._admin()
                    return self._send(200, {"object": "list", "data": list(state.adapters.values())})
                raise ApiError(404, f"no route {path}", "not_found_error")
            except ApiError as e:
                self._error(e)

        def do_DELETE(self):
            try:
                self._check_head()
                if self.path.startswith("/v1/lora_adapters/"):
                    self._admin()
                    name = self.path[len("/v1/lora_adapters/"):]
                    if name not in state.adapters:
                        raise ApiError(404, "adapter not found", "not_found_error")
                    if eng.adapter_in_use(state.adapters[name]["slot"]):
                        raise ApiError(409, f"adapter {name!r} is in use by live requests", "conflict_error")
                    eng.adapter_call(lambda bank: bank.unload(name))
                    del state.adapters[name]
                    return self._send(200, {"deleted": True, "id": name})
                raise ApiError(404, "no route", "not_found_error")
            except ApiError as e:
                self._error(e)

        def _load_adapter(self, req: dict) -> dict:
            """``POST /v1/lora_adapters {"name": ..., "path": ...}``: make a PEFT adapter resident; requests select it by
            naming it as their ``model``."""
            from ..load.lora import LoraError, load_adapter
            from ..runtime.lora_bank import LoraBankError
            name, path_ = req.get("name"), req.get("path")
            if not isinstance(name, str) or not name or not isinstance(path_, str) or not path_:
                raise ApiError(400, "`name` and `path` are required strings")
            if name == state.model_id or name in state.adapters:
                raise ApiError(409, f"the name {name!r} is already served", "conflict_error")
            try:
                adapter = load_adapter(path_, name)
                slot = eng.adapter_call(lambda bank: bank.load(adapter))
            except LookupError as e:
                raise ApiError(400, f"adapter {name!r}: {e}") from None
            except (LoraError, LoraBankError, FileNotFoundError) as e:
                raise ApiError(400, f"adapter {name!r}: {e}") from None
            state.adapters[name] = {"id": name, "object": "lora_adapter", "slot": slot, "rank": adapter.rank, "path": path_,
                                    "created": int(time.time())}
            return state.adapters[name]

        # ---- encoder routes ---------------------------------------------------------------------------------
        def _encoder_call(self, fn):
            from ..embed import EmbedError
            try:
                return eng.run(fn)
            except EmbedError as e:
                raise ApiError(400, str(e))
            except RuntimeError as e:
                raise ApiError(503, str(e), "service_unavailable")

        def _embeddings(self, req: dict) -> dict:
            inp = req.get("input")
            if isinstance(inp, str):
                inp = [inp]
            if not isinstance(inp, list) or not inp or len(inp) > 2048:
                raise ApiError(400, "`input` must be a string, a list of strings or a list of token-id lists (at most 2048)")
            fmt = req.get("encoding_format", "float")
            if fmt not in ("float", "base64"):
                raise ApiError(400, "`encoding_format` must be float or base64")
            pooling = req.get("pooling", "mean")
            emb = state.embedder
            if all(isinstance(x, str) for x in inp):
                vec, n = self._encoder_call(lambda: emb.embed(inp, pooling, bool(req.get("normalize", True))))
            elif all(isinstance(x, list) and x and all(isinstance(t, int) and 0 <= t < emb.cfg.vocab for t in x) for x in inp):
                vec = self._encoder_call(lambda: emb.embed_ids(inp, pooling, bool(req.get("normalize", True))))
                n = sum(len(x) for x in inp)
            else:
                raise ApiError(400, "`input` mixes strings and token lists, or names a token outside the vocabulary")
            dims = req.get("dimensions")
            if dims is not None:
                if not isinstance(dims, int) or not (0 < dims <= vec.shape[1]):
                    raise ApiError(400, f"`dimensions` must be between 1 and {vec.shape[1]}")
                vec = vec[:, :dims]
            def one(v):
                if fmt == "base64":
                    import base64
                    return base64.b64encode(v.astype("<f4").tobytes()).decode()
                return [float(x) for x in v]
            return {"object": "list", "model": state.model_id,
                    "data": [{"object": "embedding", "index": i, "embedding": one(v)} for i, v in enumerate(vec)],
                    "usage": {"prompt_tokens": n, "total_tokens": n}}

        def _rerank(self, req: dict) -> dict:
            q, docs = req.get("query"), req.get("documents")
            if not isinstance(q, str) or not isinstance(docs, list) or not docs or len(docs) > 1024:
                raise ApiError(400, "`query` must be a string and `documents` a non-empty list (at most 1024)")
            texts = [d if isinstance(d, str) else d.get("text") if isinstance(d, dict) else None for d in docs]
            if any(not isinstance(t, str) for t in texts):
                raise ApiError(400, "every document must be a string or an object with a `text` field")
            top_n = req.get("top_n", len(texts))
            if not isinstance(top_n, int) or top_n < 1:
                raise ApiError(400, "`top_n` must be a positive integer")
            scores, n = self._encoder_call(lambda: state.embedder.rerank(q, texts))
            order = sorted(range(len(texts)), key=lambda i: (-float(scores[i]), i))[:top_n]
            res = [{"index": i, "relevance_score": float(scores[i]),
                    **({"document": {"text": texts[i]}} if req.get("return_documents") else {})} for i in order]
            return {"model": state.model_id, "results": res, "usage": {"prompt_tokens": n, "total_tokens": n}}

        def do_POST(self):
            try:
                self._check_head()
                path = self.path.split("?")[0]
                if path in ("/v1/embeddings", "/v1/rerank"):
                    req = self._body()
                    if state.embedder is None:
                        raise ApiError(400, "the served model is a decoder: no embedding / rerank head is available")
                    if not state.limiter.allow():
                        raise ApiError(429, "rate limit exceeded", "rate_limit_error", retry_after=60)
                    return self._send(200, self._embeddings(req) if path == "/v1/embeddings" else self._rerank(req))
                if state.embedder is not None and path in ("/v1/completions", "/v1/chat/completions"):
                    self._body()
                    raise ApiError(400, "the served model is an encoder: it embeds and scores, it does not generate")
                if path == "/v1/lora_adapters":
                    self._admin()
                    return self._send(200, self._load_adapter(self._body()))
                if path not in ("/v1/completions", "/v1/chat/completions"):
                    raise ApiError(404, f"no route {path}", "not_found_error")
                if not state.limiter.allow():
                    raise ApiError(429, "rate limit exceeded", "rate_limit_error", retry_after=60)
                req = self._body()
                adapter_slot = -1
                if req.get("model") in state.adapters:       # a resident adapter is addressed as a model of its own
                    adapter_slot = state.adapters[req["model"]]["slot"]
                elif req.get("model") not in (None, state.model_id):
                    raise ApiError(404, f"model {req.get('model')!r} is not served", "not_found_error", "model")
                n = req.get("n", 1)
                if isinstance(n, bool) or not isinstance(n, int) or not (1 <= n <= 16):
                    raise ApiError(400, "n must be an integer in [1, 16]", param="n")
                chat = path.endswith("chat/completions")
                self._embeds = self._rope = None
                prompt_ids, guided_spec, tools = self._prompt(req, chat)
                embeds, rope_positions = self._embeds, self._rope
                params = sampling_from_request(req)
                jobs: List[Job] = []
                try:
                    for i in range(n):
                        sp = SamplingParams(**{**vars(params), "seed": None if params.seed is None else params.seed + i})
                        g = None
                        if guided_spec is not None:
                            g = guided_mod.build_constraint(guided_spec, eng.tk, eng.driver.eos_token, tools)
                        jobs.append(eng.submit(Job(prompt_ids, sp, stream=bool(req.get("stream")), guided=g,
                                                   adapter_slot=adapter_slot, embeds=embeds, rope_positions=rope_positions)))
                except queue.Full:
                    for j in jobs:
                        j.cancelled.set()
                    raise ApiError(429, "too many pending requests", "rate_limit_error", retry_after=1) from None
                except EngineDead as ex:
                    raise ApiError(503, f"engine unavailable: {ex}", "server_error") from None
                except guided_mod.ConstraintError as ex:
                    raise ApiError(400, str(ex)) from None
                if req.get("stream"):
                    return self._stream(jobs, chat, req)
                return self._respond(jobs, chat, req, tools)
            except ApiError as e:
                self._error(e)
            except (BrokenPipeError, ConnectionResetError, socket.timeout):
                pass

        # ---- helpers ----------------------------------------------------------------------------------------
        def _admin(self):
            auth = self.headers.get("Authorization", "")
            if state.admin_key is None or not hmac.compare_digest(auth.encode(), f"Bearer {state.admin_key}".encode()):
                raise ApiError(401, "admin key required", "authentication_error")

        def _model_obj(self):
            return {"id": state.model_id, "object": "model", "created": state.created, "owned_by": "poot-b200"}

        def _prompt(self, req: dict, chat: bool) -> Tuple[List[int], Optional[dict], Optional[list]]:
            tools = req.get("tools")
            guided_spec = None
            rf = req.get("response_format") or {}
            if rf.get("type") == "json_object":
                guided_spec = {"json": True}
            elif rf.get("type") == "json_schema":
                guided_spec = {"json_schema": (rf.get("json_schema") or {}).get("schema", {})}
            for key, kind in (("guided_choice", "choice"), ("guided_regex", "regex"), ("guided_json", "json_schema"),
                              ("guided_grammar", "grammar")):
                if req.get(key) is not None:
                    guided_spec = {kind: req[key]}
            tc = req.get("tool_choice")
            if tools and tc == "required":
                guided_spec = {"tool": None}
            elif tools and isinstance(tc, dict):
                guided_spec = {"tool": (tc.get("function") or {}).get("name")}
            if chat:
                msgs = req.get("messages")
                if not isinstance(msgs, list) or not msgs:
                    raise ApiError(400, "messages must be a non-empty list", param="messages")
                ids = self._image_prompt(msgs)
                if ids is None:
                    try:
                        text = chat_mod.render_chat(msgs, state.chat_template, state.family, True, state.bos_text,
                                                    state.eos_text, tools)
                    except chat_mod.TemplateError as ex:
                        raise ApiError(400, str(ex), param="messages") from None
                    ids = eng.tk.encode(text, add_bos=not text.startswith(state.bos_text) if state.bos_text else True)
            else:
                p = req.get("prompt")
                if isinstance(p, list) and p and all(isinstance(t, int) and not isinstance(t, bool) for t in p):
                    ids = list(p)
                elif isinstance(p, str):
                    ids = eng.tk.encode(p)
                else:
                    raise ApiError(400, "prompt must be a string or a list of token ids", param="prompt")
            if not ids:
                raise ApiError(400, "empty prompt", param="prompt")
            if len(ids) >= eng.driver.max_seq_len:
                raise ApiError(400, f"prompt of {len(ids)} tokens exceeds the context of {eng.driver.max_seq_len}")
            return ids, guided_spec, tools

        _embeds = _rope = None

        def _image_prompt(self, msgs) -> Optional[List[int]]:
            """Messages with image parts: prompt tokens with the image placeholders expanded, and the image rows staged
            for the job (``self._embeds``).  ``None`` when no message holds an image."""
            self._embeds = self._rope = None
            has = any(isinstance(m, dict) and isinstance(m.get("content"), list) and
                      any(isinstance(p, dict) and p.get("type") in ("image_url", "image", "video_url", "video") for p in m["content"]) for m in msgs)
            if not has:
                return None
            if state.vision is None:
                raise ApiError(400, "the served model takes no images: it has no vision front end", param="messages")
            try:
                if any(isinstance(p, dict) and p.get("type") in ("image", "video") for m in msgs if isinstance(m.get("content"), list)
                       for p in m["content"]):
                    raise ValueError("image and video parts are sent as image_url / video_url with a data: URL")
                ids, pixels = state.vision.prepare_messages(msgs, state.chat_template)
                self._embeds = state.vision.image_inputs(ids, pixels)
                self._rope = state.vision.rope_inputs(ids, pixels)
            except (ValueError, chat_mod.TemplateError) as ex:
                raise ApiError(400, str(ex), param="messages") from None
            return ids

        def _usage(self, jobs):
            p = len(jobs[0].prompt_tokens)
            c = sum(len(j.tokens) for j in jobs)
            return {"prompt_tokens": p, "completion_tokens": c, "total_tokens": p + c,
                    "prompt_tokens_details": {"cached_tokens": jobs[0].cached_tokens}}

        def _respond(self, jobs, chat, req, tools):
            choices = []
            for i, job in enumerate(jobs):
                try:
                    ev = job.wait(timeout=3600)
                except queue.Empty:
                    job.cancelled.set()
                    raise ApiError(408, "generation timed out", "server_error") from None
                if ev["type"] == "error":
                    for j in jobs:
                        j.cancelled.set()
                    raise ApiError(ev.get("code", 500), ev["message"], "server_error" if ev.get("code", 500) >= 500 else "invalid_request_error")
                if chat:
                    msg = {"role": "assistant", "content": job.text}
                    fr = job.finish_reason
                    if tools:
                        rest, calls = tools_mod.parse_tool_calls(job.text, "hermes")
                        if not calls and job.guided is not None:
                            try:
                                o = json.loads(job.text)
                                calls = [tools_mod._call(o["name"], o.get("arguments", {}))]
                                rest = ""
                            except (json.JSONDecodeError, KeyError, TypeError):
                                pass
                        if calls:
                            msg, fr = {"role": "assistant", "content": rest or None, "tool_calls": calls}, "tool_calls"
                    choices.append({"index": i, "message": msg, "finish_reason": fr, "logprobs": None})
                else:
                    lp = {"token_logprobs": job.logprobs, "tokens": job.tokens} if job.logprobs else None
                    choices.append({"index": i, "text": job.text, "finish_reason": job.finish_reason, "logprobs": lp})
            body = {"id": ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24],
                    "object": "chat.completion" if chat else "text_completion", "created": int(time.time()),
                    "model": state.model_id, "choices": choices, "usage": self._usage(jobs)}
            self._send(200, body)

        def _stream(self, jobs, chat, req):
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()
            self.connection.settimeout(cfg.write_timeout_secs)
            self.connection.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)   # one small write per token
            rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
            obj = "chat.completion.chunk" if chat else "text_completion"

            def send(payload):
                self.wfile.write(b"data: " + (payload if isinstance(payload, bytes) else json.dumps(payload).encode()) + b"\n\n")
                self.wfile.flush()

            try:
                if chat:
                    for i in range(len(jobs)):
                        send({"id": rid, "object": obj, "created": int(time.time()), "model": state.model_id,
                              "choices": [{"index": i, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]})
                open_jobs = set(range(len(jobs)))
                while open_jobs:
                    for i in list(open_jobs):
                        try:
                            ev = jobs[i].events.get(timeout=0.01 if len(open_jobs) > 1 else 1.0)
                        except queue.Empty:
                            continue
                        if ev["type"] == "token":
                            ch = ({"index": i, "delta": {"content": ev["text"]}, "finish_reason": None} if chat
                                  else {"index": i, "text": ev["text"], "finish_reason": None})
                            send({"id": rid, "object": obj, "created": int(time.time()), "model": state.model_id, "choices": [ch]})
                        elif ev["type"] == "done":
                            ch = ({"index": i, "delta": {}, "finish_reason": ev["finish_reason"]} if chat
                                  else {"index": i, "text": "", "finish_reason": ev["finish_reason"]})
                            send({"id": rid, "object": obj, "created": int(time.time()), "model": state.model_id, "choices": [ch]})
                            open_jobs.discard(i)
                        else:
                            send({"error": {"message": ev["message"], "type": "server_error"}})
                            open_jobs.discard(i)
                if (req.get("stream_options") or {}).get("include_usage"):
                    send({"id": rid, "object": obj, "created": int(time.time()), "model": state.model_id, "choices": [],
                          "usage": self._usage(jobs)})
                send(b"[DONE]")
            except (BrokenPipeError, ConnectionResetError, socket.timeout):
                for j in jobs:                 # the client went away: free its rows
                    j.cancelled.set()
            self.close_connection = True

    return Handler


class Server:
    def __init__(self, state: ServerState):
        host, _, port = state.cfg.addr.rpartition(":")
        self.state = state
        class _Listener(ThreadingHTTPServer):
            request_queue_size = max(128, min(state.cfg.max_connections, 1024))   # a burst of connections must not be reset
            daemon_threads = True

        self.httpd = _Listener((host, int(port)), make_handler(state))
        self.httpd.handle_error = lambda request, client_address: None   # a peer that hangs up is not news
        self.httpd.daemon_threads = True
        self.thread: Optional[threading.Thread] = None

    @property
    def port(self) -> int:
        return self.httpd.server_address[1]

    def start(self) -> None:
        self.thread = threading.Thread(target=self.httpd.serve_forever, name="poot-http", daemon=True)
        self.thread.start()

    def shutdown(self) -> None:
        """Graceful drain: stop accepting work, let live requests finish (bounded), stop the listener."""
        self.state.engine.drain(self.state.cfg.drain_timeout_secs)
        self.httpd.shutdown()
        self.httpd.server_close()
