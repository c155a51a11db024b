"""``generate``: one-shot and conversational text generation with llama-cli compatible flags.

Flag set and defaults follow crates/poot-llm/src/bin/poot/generate.rs:41-140: ``-m``, ``-p`` / ``-f``,
``--system-prompt``, ``--no-chat-template``, ``--chat-template[-file]``, ``--conversation``, ``--single-turn``,
``-n/--predict`` (-1 = until the context is full), ``-c/--ctx-size`` (0 = the model's), ``--temp`` (0), ``--top-k``
(40), ``--top-p`` (0.95), ``--min-p`` (0.05), ``--repeat-penalty`` (1.0), ``-s/--seed``, ``-r/--reverse-prompt``
(repeatable), ``--ignore-eos``, ``--backend``, ``--[no-]show-timings``, ``-v``.  Parsing is strict: an unknown
option or an out-of-range value stops before the model is loaded.
"""
from __future__ import annotations

import argparse
import sys
import time
from dataclasses import dataclass, field
from typing import List, Optional

from ..driver.sampler import SamplingParams


class _Strict(argparse.ArgumentParser):
    def error(self, message):
        raise ValueError(message)


@dataclass
class GenerateArgs:
    model: str = ""
    prompt: Optional[str] = None
    file: Optional[str] = None
    system_prompt: Optional[str] = None
    no_chat_template: bool = False
    chat_template: Optional[str] = None
    chat_template_file: Optional[str] = None
    conversation: bool = False
    single_turn: bool = False
    predict: int = -1
    ctx_size: int = 0
    temp: float = 0.0
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repeat_penalty: float = 1.0
    seed: Optional[int] = None
    reverse_prompt: List[str] = field(default_factory=list)
    ignore_eos: bool = False
    backend: str = "auto"
    lora: Optional[str] = None
    show_timings: bool = True
    verbose: bool = False

    def sampling(self, max_tokens: int) -> SamplingParams:
        return SamplingParams(temperature=self.temp, top_k=self.top_k, top_p=self.top_p, min_p=self.min_p,
                              repeat_penalty=self.repeat_penalty, seed=self.seed, max_tokens=max_tokens,
                              stop=list(self.reverse_prompt), ignore_eos=self.ignore_eos)


def parse_generate(argv: List[str]) -> GenerateArgs:
    p = _Strict(prog="poot generate", allow_abbrev=False)
    p.add_argument("-m", "--model", required=True)
    p.add_argument("-p", "--prompt")
    p.add_argument("-f", "--file")
    p.add_argument("--system-prompt")
    p.add_argument("--no-chat-template", action="store_true")
    p.add_argument("--chat-template")
    p.add_argument("--chat-template-file")
    p.add_argument("--conversation", action="store_true")
    p.add_argument("--single-turn", action="store_true")
    p.add_argument("-n", "--predict", type=int, default=-1)
    p.add_argument("-c", "--ctx-size", type=int, default=0)
    p.add_argument("--temp", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--top-p", type=float, default=0.95)
    p.add_argument("--min-p", type=float, default=0.05)
    p.add_argument("--repeat-penalty", type=float, default=1.0)
    p.add_argument("-s", "--seed", type=int)
    p.add_argument("-r", "--reverse-prompt", action="append", default=[])
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--backend", default="auto")
    p.add_argument("--lora", help="PEFT adapter directory merged into the projections at load")
    p.add_argument("--show-timings", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("-v", "--verbose", action="store_true")
    ns = p.parse_args(argv)
    a = GenerateArgs(**vars(ns))
    if a.prompt is not None and a.file is not None:
        raise ValueError("-p and -f are mutually exclusive")
    if a.prompt is None and a.file is None and not a.conversation:
        raise ValueError("a prompt is required: -p TEXT, -f FILE or --conversation")
    if a.chat_template is not None and a.chat_template_file is not None:
        raise ValueError("--chat-template and --chat-template-file are mutually exclusive")
    if a.no_chat_template and (a.chat_template or a.chat_template_file or a.system_prompt or a.conversation):
        raise ValueError("--no-chat-template excludes --chat-template, --system-prompt and --conversation")
    if a.predict < -1 or a.predict == 0:
        raise ValueError("-n must be -1 or a positive count")
    if a.ctx_size < 0 or a.temp < 0 or not (0 <= a.top_p <= 1) or not (0 <= a.min_p <= 1) or a.top_k < 0 or a.repeat_penalty <= 0:
        raise ValueError("sampling or context option out of range")
    if len(a.reverse_prompt) > 16:
        raise ValueError("at most 16 reverse prompts")
    if a.backend not in ("auto", "b200", "cuda", "fake", "oracle", "graph"):
        raise ValueError(f"--backend {a.backend!r}: this build has one device backend (b200 / cuda / auto), the CPU "
                         "`oracle` and `fake`")
    return a


def _open(a: GenerateArgs):
    from ..llm import LLM
    if a.backend == "fake" or a.model == "fake":
        return LLM.fake(rows=1, max_seq=a.ctx_size or 512)
    ctx = a.ctx_size or 4096
    if a.model.startswith("random:"):
        return LLM.random(a.model.split(":", 1)[1], rows=1, max_seq=ctx)
    if a.backend == "graph":
        # the general device executor: every traced family, equation by equation on the device
        import torch
        return LLM.graph(a.model, device="cuda" if torch.cuda.is_available() else "cpu", rows=1, max_seq=ctx, num_blocks=(ctx + 15) // 16 + 1)
    if a.backend == "oracle":
        # a GGUF's quantised matrices stay as stored: the evaluator decodes them inside its native contractions
        return LLM.oracle(a.model, rows=1, max_seq=ctx, num_blocks=(ctx + 15) // 16 + 1, lora=a.lora,
                          packed=a.model.endswith(".gguf") and not a.lora)
    return LLM.load(a.model, rows=1, max_seq=ctx, lora=a.lora)


def _template(a: GenerateArgs) -> Optional[str]:
    if a.chat_template_file:
        with open(a.chat_template_file) as f:
            return f.read()
    return a.chat_template


def run_generate(a: GenerateArgs, llm=None, out=None, inp=None) -> dict:
    """Runs the command; returns the timing record (also printed with ``--show-timings``)."""
    from ..text.chat import render_chat
    from ..text.codec import StreamDecoder
    out = out or sys.stdout
    inp = inp or sys.stdin
    t_load = time.perf_counter()
    llm = llm or _open(a)
    d, tk = llm.driver, llm.tokenizer
    load_s = time.perf_counter() - t_load
    family = llm.cfg.family if llm.cfg is not None else "llama"
    prompt = a.prompt
    if a.file:
        with open(a.file) as f:
            prompt = f.read()
    messages = [{"role": "system", "content": a.system_prompt}] if a.system_prompt else []
    timing = {"load_s": load_s, "prompt_tokens": 0, "generated": 0, "prefill_s": 0.0, "decode_s": 0.0}
    sid = None

    def one_turn(text_tokens: List[int]) -> str:
        nonlocal sid
        room = d.max_seq_len - (len(d.seqs[sid].tokens) if sid is not None else 0) - len(text_tokens)
        if room < 1:
            raise ValueError("the prompt fills the context")
        n = room if a.predict < 0 else min(a.predict, room)
        if sid is None:
            sid = d.open(text_tokens, a.sampling(n))
        else:
            d.resume(sid, text_tokens, n)
        dec, pieces, held = StreamDecoder(tk), [], ""
        t0 = time.perf_counter()
        first = None
        timing["prompt_tokens"] += len(text_tokens)
        produced = 0
        while True:
            res = [r for r in d.step([sid]) if r.token is not None]
            if not res:
                continue
            r = res[0]
            if first is None:
                first = time.perf_counter()
            d.commit(sid, [r.token])
            produced += 1
            reason = d.finished(sid, r.token)
            piece = "" if (reason == "stop" and r.token == d.eos_token) else dec.push(r.token)
            buf = held + piece
            hit = None
            for s in a.reverse_prompt:
                i = buf.find(s)
                if i >= 0 and (hit is None or i < hit):
                    hit = i
            if hit is not None:
                buf, reason = buf[:hit], reason or "stop"
                held = ""
            else:
                hold = 0
                for s in a.reverse_prompt:
                    for k in range(min(len(s) - 1, len(buf)), 0, -1):
                        if buf.endswith(s[:k]):
                            hold = max(hold, k)
                            break
                held, buf = (buf[len(buf) - hold:], buf[:len(buf) - hold]) if hold else ("", buf)
            if reason is not None and hit is None:
                buf += held + dec.flush()
            if buf:
                pieces.append(buf)
                out.write(buf)
                out.flush()
            if reason is not None:
                break
        t1 = time.perf_counter()
        timing["generated"] += produced
        timing["prefill_s"] += (first or t1) - t0
        timing["decode_s"] += t1 - (first or t1)
        return "".join(pieces)

    try:
        if a.no_chat_template:
            one_turn(tk.encode(prompt))
        elif not a.conversation:
            messages.append({"role": "user", "content": prompt})
            one_turn(tk.encode(render_chat(messages, _template(a), family, True)))
        else:
            turn = prompt
            while True:
                if turn is None:
                    out.write("\n> ")
                    out.flush()
                    turn = inp.readline()
                    if not turn:
                        break
                    turn = turn.rstrip("\n")
                    if not turn:
                        turn = None
                        continue
                before = render_chat(messages, _template(a), family, False) if messages else ""
                messages.append({"role": "user", "content": turn})
                full = render_chat(messages, _template(a), family, True)
                # only the new turn is fed: the K/V of the earlier turns stays in the sequence's blocks
                new_text = full[len(before):] if sid is not None and full.startswith(before) else full
                reply = one_turn(tk.encode(new_text, add_bos=sid is None))
                messages.append({"role": "assistant", "content": reply})
                turn = None
                if a.single_turn:
                    break
    finally:
        if sid is not None:
            d.release(sid)
    out.write("\n")
    if a.show_timings:
        pf = timing["prompt_tokens"] / timing["prefill_s"] if timing["prefill_s"] > 0 else 0.0
        dc = max(timing["generated"] - 1, 0) / timing["decode_s"] if timing["decode_s"] > 0 else 0.0
        print(f"load {timing['load_s']:.2f} s | prompt {timing['prompt_tokens']} tok, {pf:.1f} tok/s | "
              f"generated {timing['generated']} tok, {dc:.1f} tok/s", file=sys.stderr)
    return timing


def main_generate(argv: List[str]) -> int:
    try:
        a = parse_generate(argv)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    try:
        run_generate(a)
    except (ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0
