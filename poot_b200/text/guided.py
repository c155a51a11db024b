"""Guided decoding: constraints that turn the text generated so far into a per-token mask.

Constraint kinds of the reference (crates/poot-text/src/guided.rs, src/grammar.rs:1-6): a fixed ``choice`` list, a
``regex``, a ``json_schema`` (compiled to a regex for the supported subset), free-form ``json`` (a pushdown prefix
acceptor), a ``GBNF`` grammar (the stack machine llama.cpp uses) and a forced tool call (a JSON-schema constraint
built from the tool's parameters).  Every kind becomes a machine stepped over *bytes*: choice, regex, schema and tool
constraints a dense byte DFA (``text/automata.py``), free-form JSON and GBNF a stack machine whose states are immutable
values.  The mask of a step (0 = allowed, ``f32::MIN`` = excluded, the ``MASKED_LOGIT`` of the sampling rules) is the
cached allowed-token set of the machine's current state; a state's set is computed once, by a pruned walk of the
vocabulary's byte trie.  Hostile inputs are bounded: pattern length, automaton size and build work, grammar size,
nesting depth.
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


# ---- byte-level machines ----------------------------------------------------------------------------------------
JSON_GRAMMAR = r"""
root   ::= ws value ws
value  ::= object | array | string | number | "true" | "false" | "null"
object ::= "{" ws ( string ws ":" ws value ws ( "," ws string ws ":" ws value ws )* )? "}"
array  ::= "[" ws ( value ws ( "," ws value ws )* )? "]"
string ::= "\"" ( [^"\\\x00-\x1f] | "\\" ( ["\\/bfnrt] | "u" hex hex hex hex ) )* "\""
hex    ::= [0-9a-fA-F]
number ::= "-"? ( "0" | [1-9] [0-9]* ) ( "." [0-9]+ )? ( [eE] [-+]? [0-9]+ )?
ws     ::= [ \t\n\r]*
"""


class DfaMachine:
    """A regex / choice / schema constraint as a byte DFA; its states are small integers."""

    def __init__(self, dfa):
        self.dfa = dfa

    def start(self):
        return 0

    def step(self, state, byte: int):
        ns = int(self.dfa.table[state, byte])
        return None if ns < 0 else ns

    def complete(self, state) -> bool:
        return bool(self.dfa.accepting[state])

    def can_continue(self, state) -> bool:
        return bool((self.dfa.table[state] >= 0).any())

    def allowed(self, trie, state):
        return trie.walk_dfa(self.dfa, state)


class GbnfMachine:
    """The grammar's stack machine stepped over bytes.  A state is ``(set of stacks, bytes of an unfinished UTF-8
    character)``; both parts are immutable, so states are dictionary keys and stepping never copies an acceptor.  A
    character that is still incomplete is admissible when some stack top matches a character of the code-point range
    its bytes leave open."""

    def __init__(self, grammar: "Gbnf"):
        self.g = grammar
        self._helper = GbnfAcceptor(grammar, stacks=set())

    def start(self):
        return (frozenset(GbnfAcceptor(self.g).stacks), b"")

    @staticmethod
    def _open_range(prefix: bytes):
        b0, n = prefix[0], len(prefix)
        if 0xC2 <= b0 <= 0xDF:
            need, cp, bits = 2, b0 & 0x1F, 6
        elif 0xE0 <= b0 <= 0xEF:
            need, cp, bits = 3, b0 & 0x0F, 12
        elif 0xF0 <= b0 <= 0xF4:
            need, cp, bits = 4, b0 & 0x07, 18
        else:
            return None
        for c in prefix[1:]:
            if c & 0xC0 != 0x80:
                return None
            bits -= 6
            cp = (cp << 6) | (c & 0x3F)
        if n > need:
            return None
        lo = cp << bits
        hi = lo | ((1 << bits) - 1)
        # a sequence of this length encodes only code points above the shorter forms (no overlong encodings)
        floor, ceil = {2: (0x80, 0x7FF), 3: (0x800, 0xFFFF), 4: (0x10000, 0x10FFFF)}[need]
        lo, hi = max(lo, floor), min(hi, ceil)
        if lo > hi:
            return None
        return need, lo, hi

    @staticmethod
    def _matches_some(el, lo: int, hi: int) -> bool:
        _, neg, ranges = el
        rs = sorted((ord(a), ord(b)) for a, b in ranges)
        if not neg:
            return any(a <= hi and b >= lo for a, b in rs)
        cur = lo                                    # negated class: some code point of [lo, hi] outside every range
        for a, b in rs:
            if a > cur:
                break
            cur = max(cur, b + 1)
            if cur > hi:
                return False
        return cur <= hi

    def _feed_char(self, stacks, ch: str):
        nxt: set = set()
        for st in stacks:
            if st and GbnfAcceptor._match(st[-1], ch):
                self._helper._expand(st[:-1], nxt, 0)
        nxt = {st for st in nxt if len(st) <= 4 * MAX_DEPTH}      # nesting bound: deeper derivations are refused
        return (frozenset(nxt), b"") if nxt else None

    def step(self, state, byte: int):
        stacks, pend = state
        if not pend and byte < 0x80:
            return self._feed_char(stacks, chr(byte))
        pend = pend + bytes([byte])
        rng = self._open_range(pend)
        if rng is None:
            return None
        need, lo, hi = rng
        if len(pend) == need:
            try:
                ch = pend.decode("utf-8")
            except UnicodeDecodeError:
                return None
            return self._feed_char(stacks, ch)
        if not any(st and self._matches_some(st[-1], lo, hi) for st in stacks):
            return None
        return (stacks, pend)

    def complete(self, state) -> bool:
        return not state[1] and () in state[0]

    def can_continue(self, state) -> bool:
        return bool(state[1]) or any(st for st in state[0])

    def allowed(self, trie, state):
        return trie.walk(state, self.step)


# ---- constraint (machine + tokenizer) ----------------------------------------------------------------------------
_DFA_CACHE: Dict[tuple, tuple] = {}     # (kind, pattern) -> (machine, {tokenizer id: StateMasks})
_DFA_CACHE_CAP = 64


def _vocab_trie(tokenizer):
    """The tokenizer's byte trie, built once and kept on the tokenizer."""
    trie = getattr(tokenizer, "_guided_trie", None)
    if trie is None:
        from .automata import TokenTrie
        toks = []
        for t in range(tokenizer.vocab_size()):
            try:
                toks.append(bytes(tokenizer.token_bytes(t)))
            except Exception:
                toks.append(b"")
        trie = TokenTrie(toks)
        try:
            tokenizer._guided_trie = trie
        except AttributeError:
            pass
    return trie


class Constraint:
    """The state of one request under a constraint: the machine's current state, advanced by every committed token.

    ``mask`` looks the state's allowed-token set up in a cache shared by every request with the same pattern and
    tokenizer; a state seen for the first time costs one pruned walk of the vocabulary trie, a state seen before costs
    a dictionary lookup (crates/poot-text/src/guided.rs:261-350).  Tokens are bytes: a token holding half of a UTF-8
    character is allowed exactly when the machine can take those bytes."""

    def __init__(self, machine, tokenizer, eos_token: Optional[int] = None, masks=None):
        from .automata import StateMasks
        self.m, self.tk, self.eos = machine, tokenizer, eos_token
        self.state = machine.start()
        self.masks = masks if masks is not None else StateMasks()
        self._bytes: Optional[List[bytes]] = None

    def clone(self) -> "Constraint":
        c = Constraint(self.m, self.tk, self.eos, self.masks)
        c.state = self.state
        return c

    def _allowed(self, vocab: int) -> np.ndarray:
        trie = _vocab_trie(self.tk)
        st = self.state
        packed = self.masks.get(st, lambda: np.packbits(self.m.allowed(trie, st)))
        a = np.unpackbits(packed, count=trie.n_tokens).astype(bool)
        if len(a) < vocab:
            a = np.concatenate([a, np.zeros(vocab - len(a), bool)])
        return a[:vocab]

    def mask(self, vocab: int) -> np.ndarray:
        m = np.where(self._allowed(vocab), np.float32(0.0), np.float32(MASKED)).astype(np.float32)
        if self.eos is not None and self.eos < vocab:
            m[self.eos] = 0.0 if self.m.complete(self.state) else MASKED
        return m

    def feed_bytes(self, data: bytes) -> bool:
        """Advance over raw bytes (tests, prefilled text).  False when the machine dies; the state is then unchanged."""
        st = self.state
        for b in data:
            st = self.m.step(st, b)
            if st is None:
                return False
        self.state = st
        return True

    def advance(self, token: int) -> None:
        if token == self.eos:
            return
        self.feed_bytes(bytes(self.tk.token_bytes(token)))

    def done(self) -> bool:
        """True when the text is complete and nothing could extend it."""
        return self.m.complete(self.state) and not self.m.can_continue(self.state)


def _cached_dfa(kind: str, pattern: str, build):
    key = (kind, pattern)
    hit = _DFA_CACHE.get(key)
    if hit is None:
        if len(_DFA_CACHE) >= _DFA_CACHE_CAP:
            _DFA_CACHE.clear()
        hit = _DFA_CACHE[key] = (build(), {})
    return hit


def _regex_machine(pattern: str):
    from .automata import AutomatonError, ByteDfa
    if len(pattern) > MAX_PATTERN:
        raise ConstraintError("regex too long")
    try:
        return DfaMachine(ByteDfa.from_regex(pattern))
    except AutomatonError as e:
        raise ConstraintError(str(e)) from None


def build_constraint(spec: dict, tokenizer, eos_token: Optional[int] = None, tools: Optional[list] = None) -> Constraint:
    """``spec`` = {"choice": [...]} | {"regex": "..."} | {"json_schema": {...}} | {"json": true} | {"grammar": "..."} |
    {"tool": name-or-None}."""
    from .automata import ByteDfa, StateMasks
    if "choice" in spec:
        if not spec["choice"]:
            raise ConstraintError("empty choice list")
        key = "\x00".join(spec["choice"])
        machine, per_tok = _cached_dfa("choice", key, lambda: DfaMachine(ByteDfa.from_literals([c.encode("utf-8") for c in spec["choice"]])))
    elif "regex" in spec:
        machine, per_tok = _cached_dfa("regex", spec["regex"], lambda: _regex_machine(spec["regex"]))
    elif "json_schema" in spec:
        pattern = schema_to_regex(spec["json_schema"])
        machine, per_tok = _cached_dfa("regex", pattern, lambda: _regex_machine(pattern))
    elif spec.get("json"):
        machine, per_tok = _cached_dfa("gbnf", JSON_GRAMMAR, lambda: GbnfMachine(Gbnf(JSON_GRAMMAR)))
    elif "grammar" in spec:
        machine, per_tok = _cached_dfa("gbnf", spec["grammar"], lambda: GbnfMachine(Gbnf(spec["grammar"])))
    elif "tool" in spec:
        from .tools import forced_tool_schema
        pattern = schema_to_regex(forced_tool_schema(tools or [], spec["tool"]))
        machine, per_tok = _cached_dfa("regex", pattern, lambda: _regex_machine(pattern))
    else:
        raise ConstraintError("unknown constraint kind")
    masks = per_tok.setdefault(id(tokenizer), StateMasks())     # shared by every request with this pattern and tokenizer
    return Constraint(machine, tokenizer, eos_token, masks)
