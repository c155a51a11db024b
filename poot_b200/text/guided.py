"""Guided decoding: constraints that turn the text generated so far into a per-token mask.

Constraint kinds of the reference (crates/poot-text/src/guided.rs, src/grammar.rs:1-6): a fixed ``choice`` list, a
``regex``, a ``json_schema`` (compiled to a regex for the supported subset), free-form ``json`` (a pushdown prefix
acceptor), a ``GBNF`` grammar (the stack machine llama.cpp uses) and a forced tool call (a JSON-schema constraint
built from the tool's parameters).  A constraint is a character-level acceptor with ``clone`` / ``feed``; the mask
of a step marks every token whose text keeps the acceptor alive (0 = allowed, ``f32::MIN`` = excluded, the
``MASKED_LOGIT`` of the sampling rules).  Hostile inputs are bounded: pattern length, grammar size, nesting depth.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

MASKED = float(np.finfo(np.float32).min)
MAX_PATTERN = 16384
MAX_DEPTH = 64
MAX_RULES = 4096


class ConstraintError(ValueError):
    pass


# ---- acceptors -------------------------------------------------------------------------------------------------
class RegexAcceptor:
    def __init__(self, pattern: str, text: str = ""):
        import regex
        if len(pattern) > MAX_PATTERN:
            raise ConstraintError("regex too long")
        try:
            self.rx = regex.compile(pattern, flags=regex.DOTALL)
        except regex.error as e:
            raise ConstraintError(f"bad regex: {e}") from None
        self.text = text

    def clone(self):
        c = object.__new__(RegexAcceptor)
        c.rx, c.text = self.rx, self.text
        return c

    def feed(self, s: str) -> bool:
        self.text += s
        return self.rx.fullmatch(self.text, partial=True) is not None

    def complete(self) -> bool:
        return self.rx.fullmatch(self.text) is not None


class ChoiceAcceptor:
    def __init__(self, choices: Sequence[str], text: str = ""):
        if not choices:
            raise ConstraintError("empty choice list")
        self.choices, self.text = list(choices), text

    def clone(self):
        return ChoiceAcceptor(self.choices, self.text)

    def feed(self, s: str) -> bool:
        self.text += s
        return any(c.startswith(self.text) for c in self.choices)

    def complete(self) -> bool:
        return self.text in self.choices


class JsonAcceptor:
    """Prefix acceptor of one JSON value (RFC 8259) with a nesting bound."""

    def __init__(self):
        self.stack: List[str] = ["value"]     # what is expected next, innermost last
        self.buf = ""                         # scalar being read
        self.mode = None                      # None | "str" | "esc" | "num" | "lit"
        self.lit = ""
        self.uni = 0

    def clone(self):
        c = JsonAcceptor()
        c.stack, c.buf, c.mode, c.lit, c.uni = list(self.stack), self.buf, self.mode, self.lit, self.uni
        return c

    def complete(self) -> bool:
        if self.mode == "num":
            return self._num_done(self.buf) and self.stack == ["value_done_pending"]
        return not self.stack and self.mode is None

    @staticmethod
    def _num_ok_prefix(s: str) -> bool:
        import re
        return re.fullmatch(r"-?(0|[1-9]\d*)?(\.\d*)?([eE][+-]?\d*)?", s) is not None and s != ""

    @staticmethod
    def _num_done(s: str) -> bool:
        import re
        return re.fullmatch(r"-?(0|[1-9]\d*)(\.\d+)?([eE][+-]?\d+)?", s) is not None

    def _value_done(self):
        while self.stack and self.stack[-1] in ("value", "value_done_pending"):
            self.stack.pop()
            break

    def feed(self, s: str) -> bool:
        for ch in s:
            if not self._feed1(ch):
                return False
        return True

    def _feed1(self, ch: str) -> bool:
        if self.mode == "str":
            if ch == "\\":
                self.mode = "esc"
            elif ch == '"':
                self.mode = None
                self._after_string()
            elif ord(ch) < 0x20:
                return False
            return True
        if self.mode == "esc":
            if ch == "u":
                self.mode, self.uni = "uni", 4
            elif ch in '"\\/bfnrt':
                self.mode = "str"
            else:
                return False
            return True
        if self.mode == "uni":
            if ch not in "0123456789abcdefABCDEF":
                return False
            self.uni -= 1
            if self.uni == 0:
                self.mode = "str"
            return True
        if self.mode == "lit":
            self.buf += ch
            if not self.lit.startswith(self.buf):
                return False
            if self.buf == self.lit:
                self.mode = None
                self._close_value()
            return True
        if self.mode == "num":
            if self._num_ok_prefix(self.buf + ch):
                self.buf += ch
                return True
            if not self._num_done(self.buf):
                return False
            self.mode = None
            self.stack.pop()          # value_done_pending
            self._close_value(pop=False)
            return self._feed1(ch)
        if ch in " \t\r\n":
            return True
        if not self.stack:
            return False
        top = self.stack[-1]
        if top == "value" or top == "value_or_end_array":
            if top == "value_or_end_array":
                if ch == "]":
                    self.stack.pop()
                    self._close_value(pop=False)
                    return True
                self.stack[-1] = "array_next"
                self.stack.append("value")
            return self._start_value(ch)
        if top == "key_or_end":
            if ch == "}":
                self.stack.pop()
                self._close_value(pop=False)
                return True
            if ch == '"':
                self.stack[-1] = "colon"
                self.mode = "str"
                self.stack.append("keystr")
                return True
            return False
        if top == "key":
            if ch == '"':
                self.stack[-1] = "colon"
                self.mode = "str"
                self.stack.append("keystr")
                return True
            return False
        if top == "colon":
            if ch == ":":
                self.stack[-1] = "object_next"
                self.stack.append("value")
                return True
            return False
        if top == "object_next":
            if ch == ",":
                self.stack[-1] = "key"
                return True
            if ch == "}":
                self.stack.pop()
                self._close_value(pop=False)
                return True
            return False
        if top == "array_next":
            if ch == ",":
                self.stack.append("value")
                return True
            if ch == "]":
                self.stack.pop()
                self._close_value(pop=False)
                return True
            return False
        return False

    def _after_string(self):
        if self.stack and self.stack[-1] == "keystr":
            self.stack.pop()
        else:
            self._close_value()

    def _close_value(self, pop: bool = True):
        if pop and self.stack and self.stack[-1] == "value":
            self.stack.pop()

    def _start_value(self, ch: str) -> bool:
        if len(self.stack) > MAX_DEPTH:
            return False
        if ch == "{":
            self.stack[-1] = "key_or_end"
            return True
        if ch == "[":
            self.stack[-1] = "value_or_end_array"
            return True
        if ch == '"':
            self.mode = "str"
            return True
        if ch in "-0123456789":
            self.mode, self.buf = "num", ch
            self.stack[-1] = "value_done_pending"
            return True
        for lit in ("true", "false", "null"):
            if ch == lit[0]:
                self.mode, self.lit, self.buf = "lit", lit, ch
                return True
        return False


# ---- JSON schema -> regex (supported subset) -------------------------------------------------------------------
_WS = r"[ \n\t]*"
_STR = r'"(?:[^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})*"'
_NUM = r"-?(?:0|[1-9][0-9]*)(?:\.[0-9]+)?(?:[eE][+-]?[0-9]+)?"
_INT = r"-?(?:0|[1-9][0-9]*)"


def schema_to_regex(schema: dict, depth: int = 0) -> str:
    import regex
    if depth > MAX_DEPTH:
        raise ConstraintError("schema nests too deeply")
    if "const" in schema:
        return regex.escape(json.dumps(schema["const"]))
    if "enum" in schema:
        return "(?:" + "|".join(regex.escape(json.dumps(v)) for v in schema["enum"]) + ")"
    if "anyOf" in schema or "oneOf" in schema:
        return "(?:" + "|".join(schema_to_regex(s, depth + 1) for s in schema.get("anyOf", schema.get("oneOf"))) + ")"
    t = schema.get("type")
    if isinstance(t, list):
        return "(?:" + "|".join(schema_to_regex({**schema, "type": x}, depth + 1) for x in t) + ")"
    if t == "string":
        if "pattern" in schema:
            return '"' + schema["pattern"].lstrip("^").rstrip("$") + '"'
        return _STR
    if t == "integer":
        return _INT
    if t == "number":
        return _NUM
    if t == "boolean":
        return "(?:true|false)"
    if t == "null":
        return "null"
    if t == "array":
        item = schema_to_regex(schema.get("items", {}), depth + 1) if schema.get("items") else _any_value(depth + 1)
        lo, hi = schema.get("minItems", 0), schema.get("maxItems")
        rest = f"(?:{_WS},{_WS}{item})"
        if hi is not None:
            body = f"{item}{rest}{{{max(lo - 1, 0)},{hi - 1}}}" if hi > 0 else ""
        else:
            body = f"{item}{rest}{{{max(lo - 1, 0)},}}"
        if lo == 0:
            body = f"(?:{body})?" if body else ""
        return rf"\[{_WS}{body}{_WS}\]"
    if t == "object" or "properties" in schema:
        props = schema.get("properties", {})
        if not props:
            return rf"\{{{_WS}(?:{_STR}{_WS}:{_WS}{_any_value(depth + 1)}(?:{_WS},{_WS}{_STR}{_WS}:{_WS}{_any_value(depth + 1)})*)?{_WS}\}}"
        req = set(schema.get("required", props.keys()))
        parts = []
        for k, sub in props.items():
            item = rf'"{regex.escape(k)}"{_WS}:{_WS}{schema_to_regex(sub, depth + 1)}'
            parts.append((item, k in req))
        # properties appear in declaration order; optional ones may be omitted
        out, first = "", True
        for item, required in parts:
            sep = "" if first else rf"{_WS},{_WS}"
            piece = sep + item
            if required:
                out += piece
                first = False
            else:
                out += f"(?:{piece})?" if not first else f"(?:{item}{_WS},{_WS})?"
        return rf"\{{{_WS}{out}{_WS}\}}"
    return _any_value(depth + 1)


def _any_value(depth: int) -> str:
    if depth > 3:
        return rf"(?:{_STR}|{_NUM}|true|false|null)"
    inner = _any_value(depth + 1)
    return (rf"(?:{_STR}|{_NUM}|true|false|null|\[{_WS}(?:{inner}(?:{_WS},{_WS}{inner})*)?{_WS}\]|"
            rf"\{{{_WS}(?:{_STR}{_WS}:{_WS}{inner}(?:{_WS},{_WS}{_STR}{_WS}:{_WS}{inner})*)?{_WS}\}})")


# ---- GBNF ------------------------------------------------------------------------------------------------------
class Gbnf:
    """Parsed grammar: rule name -> alternatives -> elements; an element is ("chars", negated, ranges) or
    ("ref", rule) ; repetition operators are desugared into helper rules."""

    def __init__(self, text: str):
        if len(text) > 4 * MAX_PATTERN:
            raise ConstraintError("grammar too long")
        self.rules: Dict[str, List[List[tuple]]] = {}
        self._n = 0
        self._parse(text)
        if "root" not in self.rules:
            raise ConstraintError("grammar has no root rule")
        for alts in self.rules.values():
            for alt in alts:
                for el in alt:
                    if el[0] == "ref" and el[1] not in self.rules:
                        raise ConstraintError(f"undefined rule {el[1]!r}")

    def _fresh(self, base: str) -> str:
        self._n += 1
        if self._n > MAX_RULES:
            raise ConstraintError("grammar too large")
        return f"{base}_{self._n}"

    def _parse(self, text: str) -> None:
        self.s, self.i = text, 0
        while True:
            self._ws(True)
            if self.i >= len(self.s):
                break
            name = self._name()
            self._ws(False)
            if self.s[self.i:self.i + 3] != "::=":
                raise ConstraintError(f"expected ::= after {name!r}")
            self.i += 3
            self.rules[name] = self._alts(name)

    def _ws(self, newlines: bool) -> None:
        while self.i < len(self.s):
            c = self.s[self.i]
            if c == "#":
                while self.i < len(self.s) and self.s[self.i] != "\n":
                    self.i += 1
            elif c in " \t" or (newlines and c in "\r\n"):
                self.i += 1
            elif c in "\r\n" and not newlines:
                # a newline continues the rule only when the next non-blank token is '|'
                j = self.i
                while j < len(self.s) and self.s[j] in " \t\r\n":
                    j += 1
                if j < len(self.s) and self.s[j] == "|":
                    self.i = j
                else:
                    return
            else:
                return

    def _name(self) -> str:
        j = self.i
        while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "-_"):
            j += 1
        if j == self.i:
            raise ConstraintError(f"expected a rule name at offset {self.i}")
        name, self.i = self.s[self.i:j], j
        return name

    def _alts(self, rule: str) -> List[List[tuple]]:
        alts = [self._seq(rule)]
        self._ws(False)
        while self.i < len(self.s) and self.s[self.i] == "|":
            self.i += 1
            alts.append(self._seq(rule))
            self._ws(False)
        return alts

    def _char(self) -> str:
        c = self.s[self.i]
        if c == "\\":
            n = self.s[self.i + 1]
            self.i += 2
            if n == "x":
                v = chr(int(self.s[self.i:self.i + 2], 16)); self.i += 2
                return v
            if n == "u":
                v = chr(int(self.s[self.i:self.i + 4], 16)); self.i += 4
                return v
            return {"n": "\n", "r": "\r", "t": "\t"}.get(n, n)
        self.i += 1
        return c

    def _seq(self, rule: str) -> List[tuple]:
        seq: List[tuple] = []
        while True:
            self._ws(False)
            if self.i >= len(self.s):
                break
            c = self.s[self.i]
            last_start = len(seq)
            if c == '"':
                self.i += 1
                while self.s[self.i] != '"':
                    ch = self._char()
                    seq.append(("chars", False, ((ch, ch),)))
                self.i += 1
            elif c == "[":
                self.i += 1
                neg = self.s[self.i] == "^"
                if neg:
                    self.i += 1
                ranges = []
                while self.s[self.i] != "]":
                    lo = self._char()
                    hi = lo
                    if self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                        self.i += 1
                        hi = self._char()
                    ranges.append((lo, hi))
                self.i += 1
                seq.append(("chars", neg, tuple(ranges)))
            elif c == "(":
                self.i += 1
                sub = self._fresh(rule)
                self.rules[sub] = self._alts(rule)
                self._ws(True)
                if self.s[self.i] != ")":
                    raise ConstraintError("expected )")
                self.i += 1
                seq.append(("ref", sub))
            elif c == ".":
                self.i += 1
                seq.append(("chars", True, ()))
            elif c.isalnum() or c in "-_":
                seq.append(("ref", self._name()))
            else:
                break
            if self.i < len(self.s) and self.s[self.i] in "*+?":
                op = self.s[self.i]
                self.i += 1
                item = seq[last_start:]
                del seq[last_start:]
                sub = self._fresh(rule)
                if op == "*":
                    self.rules[sub] = [item + [("ref", sub)], []]
                elif op == "+":
                    self.rules[sub] = [item + [("ref", sub)], item]
                else:
                    self.rules[sub] = [item, []]
                seq.append(("ref", sub))
        return seq


class GbnfAcceptor:
    """Set of stacks of pending elements (llama.cpp's grammar machine)."""

    def __init__(self, grammar: Gbnf, stacks=None):
        self.g = grammar
        if stacks is None:
            stacks = set()
            for alt in grammar.rules["root"]:
                self._expand(tuple(reversed(alt)), stacks, 0)
        self.stacks = stacks

    def clone(self):
        return GbnfAcceptor(self.g, set(self.stacks))

    def _expand(self, stack: tuple, out: set, depth: int) -> None:
        """Resolve rule references on top of the stack until a terminal (or the empty stack) is on top."""
        if depth > 4 * MAX_DEPTH or len(out) > 8192:
            return
        if not stack or stack[-1][0] == "chars":
            out.add(stack)
            return
        _, name = stack[-1]
        for alt in self.g.rules[name]:
            self._expand(stack[:-1] + tuple(reversed(alt)), out, depth + 1)

    @staticmethod
    def _match(el, ch: str) -> bool:
        _, neg, ranges = el
        hit = any(lo <= ch <= hi for lo, hi in ranges)
        return hit != neg

    def feed(self, s: str) -> bool:
        for ch in s:
            nxt: set = set()
            for st in self.stacks:
                if st and self._match(st[-1], ch):
                    self._expand(st[:-1], nxt, 0)
            self.stacks = nxt
            if not nxt:
                return False
        return True

    def complete(self) -> bool:
        return () in self.stacks


# ---- constraint (acceptor + tokenizer) -------------------------------------------------------------------------
class Constraint:
    def __init__(self, acceptor, tokenizer, eos_token: Optional[int] = None):
        self.acc, self.tk, self.eos = acceptor, tokenizer, eos_token
        self._texts: Optional[List[str]] = None
        self._by_first: Dict[str, List[int]] = {}

    def _table(self, vocab: int) -> List[str]:
        if self._texts is None:
            self._texts = []
            for t in range(vocab):
                try:
                    s = self.tk.token_bytes(t).decode("utf-8")
                except UnicodeDecodeError:
                    s = ""
                self._texts.append(s)
                if s:
                    self._by_first.setdefault(s[0], []).append(t)
        return self._texts

    def mask(self, vocab: int) -> np.ndarray:
        texts = self._table(vocab)
        m = np.full(vocab, MASKED, dtype=np.float32)
        for first, toks in self._by_first.items():
            if not self.acc.clone().feed(first):
                continue                                   # no token starting with this character can continue
            for t in toks:
                s = texts[t]
                if len(s) == 1 or self.acc.clone().feed(s):
                    m[t] = 0.0
        if self.eos is not None and self.acc.complete():
            m[self.eos] = 0.0
        return m

    def advance(self, token: int) -> None:
        if token == self.eos:
            return
        texts = self._table(max(self.tk.vocab_size(), token + 1))
        self.acc.feed(texts[token])

    def done(self) -> bool:
        """True when the text is complete and no token could extend it."""
        if not self.acc.complete():
            return False
        texts = self._texts or []
        return not any(self.acc.clone().feed(c) for c in self._by_first)


def build_constraint(spec: dict, tokenizer, eos_token: Optional[int] = None, tools: Optional[list] = None) -> Constraint:
    """``spec`` = {"choice": [...]} | {"regex": "..."} | {"json_schema": {...}} | {"json": true} | {"grammar": "..."} |
    {"tool": name-or-None}."""
    if "choice" in spec:
        acc = ChoiceAcceptor(spec["choice"])
    elif "regex" in spec:
        acc = RegexAcceptor(spec["regex"])
    elif "json_schema" in spec:
        acc = RegexAcceptor(schema_to_regex(spec["json_schema"]))
    elif spec.get("json"):
        acc = JsonAcceptor()
    elif "grammar" in spec:
        acc = GbnfAcceptor(Gbnf(spec["grammar"]))
    elif "tool" in spec:
        from .tools import forced_tool_schema
        acc = RegexAcceptor(schema_to_regex(forced_tool_schema(tools or [], spec["tool"])))
    else:
        raise ConstraintError("unknown constraint kind")
    return Constraint(acc, tokenizer, eos_token)
