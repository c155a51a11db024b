"""The engine thread: one continuous-batching loop over the driver.

One iteration (crates/poot-serve/src/batch/engine.rs:579-830): intake new jobs -> release cancelled -> fail jobs
that waited too long -> admit (oldest first, while rows and KV blocks remain; nothing is preempted) -> ONE driver
step over every live sequence (decode rows reserved first, prefill pieces bin-packed into the token budget) ->
commit tokens (EOS / stop strings / max_tokens), stream each kept token over the job's bounded channel -> finish
and release -> refresh gauges.  A refused step fails only its requests; a fault kills the engine and ``/health``
turns ``503 dead`` (website/docs/serve/continuous-batching.md:30-34).
"""
from __future__ import annotations

import queue
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from ..driver.driver import Driver, DriverError, NoFreeRow, SamplerFault
from ..driver.kvcache import OutOfBlocks
from ..driver.sampler import SamplingParams
from ..text.codec import StreamDecoder
from .metrics import Metrics


@dataclass
class Job:
    prompt_tokens: List[int]
    params: SamplingParams
    stream: bool = False
    guided: Optional[object] = None
    adapter_slot: int = -1             # resident LoRA adapter the request selected (-1 = base model)
    embeds: Optional[tuple] = None     # (positions, rows): rows that replace the embeddings of those prompt tokens (image rows)
    rope_positions: Optional[object] = None   # [3, prompt] rotary position streams of a sectioned rope (None: the positions)
    id: int = 0
    created: float = field(default_factory=time.monotonic)
    events: "queue.Queue" = field(default_factory=lambda: queue.Queue(maxsize=4096))
    cancelled: threading.Event = field(default_factory=threading.Event)
    # filled by the engine
    seq_id: Optional[int] = None
    text: str = ""
    tokens: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    first_token_at: Optional[float] = None
    last_token_at: Optional[float] = None
    admitted_at: Optional[float] = None
    cached_tokens: int = 0
    decoder: Optional[StreamDecoder] = None
    held: str = ""                     # text withheld while it could still be the start of a stop string

    def wait(self, timeout: Optional[float] = None):
        """Block until the job ends; returns the final event."""
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            left = None if deadline is None else max(0.0, deadline - time.monotonic())
            ev = self.events.get(timeout=left)
            if ev["type"] in ("done", "error"):
                return ev


class EngineDead(RuntimeError):
    pass


class ServeEngine:
    def __init__(self, driver: Driver, tokenizer, metrics: Optional[Metrics] = None, max_pending: int = 256,
                 max_queue_wait: float = 60.0, on_step: Optional[Callable] = None, draft=None, timing=None,
                 step_deadline: Optional[float] = None):
        self.driver, self.tk = driver, tokenizer
        self.metrics = metrics or Metrics()
        self.inbox: "queue.Queue[Job]" = queue.Queue()
        self.max_pending, self.max_queue_wait = max_pending, max_queue_wait
        self.waiting: List[Job] = []
        self.live: Dict[int, Job] = {}       # seq_id -> job
        self.state = "starting"              # starting | serving | draining | dead
        self.cause: Optional[str] = None
        self._ids = 0
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.on_step = on_step
        self._memory_roles = None
        self.draft = draft                   # draft policy (``propose(tokens)``) used while one greedy sequence is live
        self.timing = timing                 # profile.TimingSnapshot, or None: counters only
        self.busy_s = 0.0
        self._admin: "queue.Queue" = queue.Queue()
        # step-deadline watchdog: a step that is still running after this many seconds is declared lost
        self.step_deadline = step_deadline
        self._step_started: Optional[float] = None
        self._watchdog: Optional[threading.Thread] = None
        self.metrics.set("poot_slot_capacity", driver.max_rows)

    # ---- submission (any thread) -------------------------------------------------------------------------------
    def pending(self) -> int:
        return self.inbox.qsize() + len(self.waiting)

    def submit(self, job: Job) -> Job:
        if self.state == "dead":
            raise EngineDead(self.cause or "engine is dead")
        if self.state == "draining":
            raise EngineDead("draining")
        if self.pending() >= self.max_pending:
            self.metrics.inc("poot_requests_rejected_total")
            raise queue.Full()
        with self._lock:
            self._ids += 1
            job.id = self._ids
        job.decoder = StreamDecoder(self.tk)
        self.metrics.inc("poot_requests_total")
        self.inbox.put(job)
        return job

    # ---- resident adapters (admin thread; serialised with the engine thread by the admin queue) -----------------
    @property
    def adapter_bank(self):
        inner = getattr(self.driver.engine, "inner", self.driver.engine)
        return getattr(getattr(inner, "e", None), "lora", None)

    def adapter_call(self, fn):
        """Run ``fn(bank)`` on the engine thread between two steps (the bank must not change under a running step)."""
        if self.adapter_bank is None:
            raise LookupError("adapter serving is not enabled (start the server with --lora-slots N)")
        box: "queue.Queue" = queue.Queue(maxsize=1)
        self._admin.put((fn, box))
        if self._thread is None or not self._thread.is_alive():       # no engine thread (tests drive iteration() themselves)
            self._run_admin()
        ok, val = box.get(timeout=60)
        if not ok:
            raise val
        return val

    def _run_admin(self) -> None:
        while True:
            try:
                fn, box = self._admin.get_nowait()
            except queue.Empty:
                return
            try:
                box.put((True, fn(self.adapter_bank)))
            except Exception as e:      # reported to the admin caller, the engine keeps serving
                box.put((False, e))

    def adapter_in_use(self, slot: int) -> bool:
        return any(j.adapter_slot == slot for j in list(self.live.values()) + list(self.waiting))

    # ---- lifecycle ---------------------------------------------------------------------------------------------
    def start(self) -> None:
        self.state = "serving"
        self._thread = threading.Thread(target=self._run_guarded, name="poot-engine", daemon=True)
        self._thread.start()
        if self.step_deadline:
            self._watchdog = threading.Thread(target=self._watch_steps, name="poot-step-watchdog", daemon=True)
            self._watchdog.start()

    def _watch_steps(self) -> None:
        """A step that outlives ``step_deadline`` cannot be interrupted from here, but the engine can be told to give
        up: ``abort()`` sets the device's abort word (every wait on another rank returns at once) and, on a multi-rank
        engine, tells the followers to stop.  The engine is dead from then on: requests in flight fail, new ones get
        503 with the cause, and the blocked step ends with a typed error when its kernels have drained."""
        while not self._stop.is_set() and self.state != "dead":
            t0 = self._step_started
            if t0 is not None and time.monotonic() - t0 > self.step_deadline:
                self.state, self.cause = "dead", f"fault: a step exceeded its deadline of {self.step_deadline:.1f} s"
                self.metrics.inc("poot_step_deadline_exceeded_total")
                abort = getattr(self.driver.engine, "abort", None)
                if abort is not None:
                    try:
                        abort()
                    except Exception:
                        traceback.print_exc()
                for job in list(self.live.values()) + list(self.waiting):
                    self._fail(job, "engine fault: step deadline exceeded")
                return
            self._stop.wait(min(0.05, self.step_deadline / 4))

    def drain(self, timeout: float = 30.0) -> None:
        """Stop admitting, let live requests finish (bounded), then stop the thread."""
        if self.state == "serving":
            self.state = "draining"
        deadline = time.monotonic() + timeout
        while (self.live or self.waiting or not self.inbox.empty()) and time.monotonic() < deadline and self.state != "dead":
            time.sleep(0.01)
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def _run_guarded(self) -> None:
        try:
            self.run()
        except Exception as e:   # a fault, not a refusal: the engine is dead from here on
            if self.state != "dead":     # the watchdog may have named the cause already
                self.state, self.cause = "dead", f"fault: {e}"
            traceback.print_exc()
            for job in list(self.live.values()) + self.waiting:
                self._fail(job, "engine fault")
            self.live.clear()
            self.waiting.clear()

    def run(self) -> None:
        while not self._stop.is_set():
            worked = self.iteration()
            if not worked:
                try:
                    job = self.inbox.get(timeout=0.02)
                    self.waiting.append(job)
                except queue.Empty:
                    pass

    # ---- one loop iteration ------------------------------------------------------------------------------------
    def iteration(self) -> bool:
        d, m = self.driver, self.metrics
        self._run_admin()
        while True:                                     # intake
            try:
                self.waiting.append(self.inbox.get_nowait())
            except queue.Empty:
                break
        for sid, job in list(self.live.items()):        # release cancelled
            if job.cancelled.is_set():
                d.release(sid, "preempted")
                del self.live[sid]
                m.inc("poot_requests_cancelled_total")
                job.events.put({"type": "done", "finish_reason": "cancelled"})
        now = time.monotonic()
        keep = []
        for job in self.waiting:                        # fail overdue / drop cancelled
            if job.cancelled.is_set():
                m.inc("poot_requests_cancelled_total")
                job.events.put({"type": "done", "finish_reason": "cancelled"})
            elif now - job.created > self.max_queue_wait:
                self._fail(job, "queue wait timeout", code=503)
            else:
                keep.append(job)
        self.waiting = keep
        while self.waiting and self.state in ("serving", "draining"):   # admit oldest first
            job = self.waiting[0]
            try:
                sid = d.open(job.prompt_tokens, job.params, guided=job.guided, adapter_slot=job.adapter_slot,
                             embeds=job.embeds, rope_positions=job.rope_positions)
            except (NoFreeRow, OutOfBlocks):
                if not self.live and not d.seqs:        # can never fit
                    self.waiting.pop(0)
                    self._fail(job, "request does not fit the KV capacity", code=400)
                    continue
                break
            except (DriverError, ValueError) as e:
                self.waiting.pop(0)
                self._fail(job, str(e), code=400)
                continue
            self.waiting.pop(0)
            job.seq_id, job.admitted_at = sid, time.monotonic()
            job.cached_tokens = d.seqs[sid].cached_tokens
            m.observe("poot_queue_wait_ms", (job.admitted_at - job.created) * 1e3)
            m.inc("poot_prompt_tokens_total", len(job.prompt_tokens))
            self.live[sid] = job
        if not self.live:
            self._gauges()
            return False
        t0 = time.monotonic()
        if self.draft is not None and len(self.live) == 1 and self._speculate():
            self.busy_s += time.monotonic() - t0
            self._gauges()
            return True
        self._step_started = t0
        try:
            results = d.step(list(self.live))
        except SamplerFault as e:                       # fails only its request
            job = self.live.pop(e.seq_id)
            d.release(e.seq_id, "preempted")
            self._fail(job, str(e), code=500)
            return True
        finally:
            self._step_started = None
        if self.state == "dead":                        # the watchdog gave this step up: its tokens are not committed
            raise EngineDead(self.cause or "engine is dead")
        step_s = time.monotonic() - t0
        self.busy_s += step_s
        if self.timing is not None:
            eng = d.engine
            run_ms = getattr(eng, "last_run_ms", None)
            host = {"step": step_s * 1e3}
            if run_ms is not None:
                host = {"plan": max(step_s * 1e3 - run_ms, 0.0), "run": run_ms}
            self.timing.record_step(sum(r.consumed for r in results), len(results), host,
                                    getattr(eng, "last_device_ms", None))
            self.timing.counters.dispatches += getattr(eng, "last_launches", 0) or 0
            self.timing.counters.replays += 1
        m.inc("poot_engine_steps_total")
        m.set("poot_batch_size", len(results))
        if self.on_step is not None:
            self.on_step(results)
        for r in results:
            if r.token is None:
                continue
            job = self.live[r.seq_id]
            self._commit(job, r)
        self._gauges()
        return True

    def _speculate(self) -> bool:
        """Draft-and-verify for a lone greedy sequence (speculation gives nothing once rows batch together)."""
        from ..driver.driver import RowResult
        from ..driver.speculate import speculative_step
        d = self.driver
        sid, job = next(iter(self.live.items()))
        s = d.seqs[sid]
        sp = s.params
        if s.pending != 1 or s.generated == 0 or not sp.greedy or s.guided is not None or sp.needs_adjust or sp.logprobs:
            return False
        toks = speculative_step(d, sid, self.draft)
        self.metrics.inc("poot_engine_steps_total")
        self.metrics.set("poot_batch_size", 1)
        for t in toks:
            self._commit(job, RowResult(sid, t, 1, None))
            if sid not in self.live:
                break
        return True

    def _commit(self, job: Job, r) -> None:
        d, m = self.driver, self.metrics
        now = time.monotonic()
        d.commit(r.seq_id, [r.token])
        job.tokens.append(r.token)
        if r.logprob is not None:
            job.logprobs.append(r.logprob)
        if job.first_token_at is None:
            job.first_token_at = now
            m.observe("poot_ttft_ms", (now - job.created) * 1e3)
        else:
            m.observe("poot_itl_ms", (now - job.last_token_at) * 1e3)
        job.last_token_at = now
        m.inc("poot_completion_tokens_total")
        reason = d.finished(r.seq_id, r.token)
        piece = "" if (reason == "stop" and r.token == d.eos_token) else job.decoder.push(r.token)
        emit, hit = self._stop_strings(job, piece)
        if hit:
            reason = "stop"
        if reason is not None:
            if not hit:
                emit += job.held + job.decoder.flush()
                job.held = ""
        if emit:
            job.text += emit
            if job.stream:
                self._put(job, {"type": "token", "text": emit, "token": r.token, "logprob": r.logprob})
        if reason is not None:
            info = d.release(r.seq_id, "finished")
            del self.live[r.seq_id]
            job.finish_reason = reason
            m.inc("poot_requests_completed_total")
            m.observe("poot_request_e2e_ms", (now - job.created) * 1e3)
            m.inc("poot_prefix_cache_hit_tokens_total", info["cached_tokens"])
            m.inc("poot_prefix_cache_query_tokens_total", len(job.prompt_tokens))
            self._put(job, {"type": "done", "finish_reason": reason})

    def _stop_strings(self, job: Job, piece: str):
        """Returns (text safe to emit, whether a stop string completed).  Text that could still become a stop string
        is held back; the stop string itself is never emitted."""
        stops = job.params.stop
        if not stops:
            return piece, False
        buf = job.held + piece
        for s in stops:
            i = buf.find(s)
            if i >= 0:
                job.held = ""
                return buf[:i], True
        hold = 0
        for s in stops:
            for n in range(min(len(s) - 1, len(buf)), 0, -1):
                if buf.endswith(s[:n]):
                    hold = max(hold, n)
                    break
        job.held = buf[len(buf) - hold:] if hold else ""
        return buf[:len(buf) - hold] if hold else buf, False

    def _put(self, job: Job, ev: dict) -> None:
        try:
            job.events.put(ev, timeout=5.0)
        except queue.Full:        # the client stopped reading: treat as cancelled
            job.cancelled.set()

    def _fail(self, job: Job, msg: str, code: int = 500) -> None:
        job.error = msg
        self.metrics.inc("poot_requests_errored_total")
        try:
            job.events.put_nowait({"type": "error", "message": msg, "code": code})
        except queue.Full:
            pass

    def _gauges(self) -> None:
        m, d = self.metrics, self.driver
        kv = d.kv_usage()
        m.set("poot_inflight_requests", len(self.live))
        m.set("poot_queue_depth", len(self.waiting) + self.inbox.qsize())
        m.set("poot_kv_usage_ratio", kv["usage_ratio"])
        m.set("poot_kv_blocks_used", kv["blocks_used"])
        m.set("poot_kv_blocks_total", kv["blocks_total"])
        up = max(time.time() - m.started, 1e-9)
        m.set("poot_gpu_active_ratio", min(1.0, self.busy_s / up))
        if self._memory_roles is None:          # bytes by buffer role: fixed once the engine is built, counted once
            self._memory_roles = {}
            inner = getattr(d.engine, "inner", d.engine)
            eng = getattr(inner, "e", None)
            if eng is not None and hasattr(eng, "kv"):
                from ..profile.memory import account
                self._memory_roles = account(eng, inner).bytes_by_role
            for role, n in self._memory_roles.items():
                m.set(f"poot_memory_{role}_bytes", n)

    def health(self) -> dict:
        h = {"status": self.state}
        if self.state == "dead":
            h["cause"] = self.cause
        if self.state == "serving":
            h.update({"backend": "b200", "rows": self.driver.max_rows, "max_seq": self.driver.max_seq_len})
        return h
