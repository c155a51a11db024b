"""Byte-level automata for guided decoding: regex -> NFA -> DFA over UTF-8 bytes, a token trie, and cached per-state
token masks.

A regex constraint is compiled once into a dense DFA over *bytes* (a Thompson NFA from the parsed pattern, code-point
classes expanded to UTF-8 byte sequences, subset construction over byte equivalence classes).  States from which no
accepting state can be reached are dead, so "the output is still a prefix of some full match" is exactly "the DFA is
not dead".  The vocabulary is a trie of the tokens' bytes; the allowed-token mask of a DFA state is one pruned walk of
that trie (in the C++ host library when it is built), computed on the first visit of the state and cached, so a decode
step costs a dictionary lookup - not a regex match per vocabulary entry.  Tokens are handled as bytes: a token that is
only part of a UTF-8 character is allowed exactly when the automaton can take those bytes.

This is the structure of the reference's constraint (crates/poot-text/src/guided.rs:261-350: byte DFA, ``StateMasks``
cache keyed by DFA state, size limits on the automaton) built without a regex-automata library.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

MAX_NFA_STATES = 50_000
MAX_DFA_STATES = 20_000
MAX_DFA_WORK = 20_000_000      # edge tests of the subset construction: a hostile pattern is refused in about a second
STATE_MASK_CAP = 4096
MAX_CODEPOINT = 0x10FFFF


class AutomatonError(ValueError):
    """The pattern uses a construct that has no finite byte automaton here, or the automaton would be too large."""


# ---- UTF-8 ranges ------------------------------------------------------------------------------------------------
def utf8_sequences(lo: int, hi: int):
    """Sequences of byte ranges that together match exactly the code points ``lo..hi`` (surrogates excluded)."""
    stack = [(lo, hi)]
    while stack:
        lo, hi = stack.pop()
        if lo > hi:
            continue
        if lo <= 0xDFFF and hi >= 0xD800:              # cut the surrogate block out
            stack.append((lo, 0xD7FF))
            stack.append((0xE000, hi))
            continue
        split = next((mx for mx in (0x7F, 0x7FF, 0xFFFF) if lo <= mx < hi), None)
        if split is not None:
            stack.append((lo, split))
            stack.append((split + 1, hi))
            continue
        if hi <= 0x7F:
            yield [(lo, hi)]
            continue
        done = False
        for i in (1, 2, 3):
            m = (1 << (6 * i)) - 1
            if (lo & ~m) != (hi & ~m):
                if lo & m:
                    stack.append((lo, lo | m))
                    stack.append(((lo | m) + 1, hi))
                    done = True
                    break
                if (hi & m) != m:
                    stack.append((lo, (hi & ~m) - 1))
                    stack.append((hi & ~m, hi))
                    done = True
                    break
        if done:
            continue
        a, b = chr(lo).encode("utf-8"), chr(hi).encode("utf-8")
        yield list(zip(a, b))


def _merge(ranges: Iterable[Tuple[int, int]]) -> List[Tuple[int, int]]:
    out: List[Tuple[int, int]] = []
    for lo, hi in sorted(ranges):
        if out and lo <= out[-1][1] + 1:
            out[-1] = (out[-1][0], max(out[-1][1], hi))
        else:
            out.append((lo, hi))
    return out


def _complement(ranges: List[Tuple[int, int]]) -> List[Tuple[int, int]]:
    out, nxt = [], 0
    for lo, hi in _merge(ranges):
        if lo > nxt:
            out.append((nxt, lo - 1))
        nxt = hi + 1
    if nxt <= MAX_CODEPOINT:
        out.append((nxt, MAX_CODEPOINT))
    return out


_CATEGORIES = {
    "CATEGORY_DIGIT": [(48, 57)], "CATEGORY_SPACE": [(9, 13), (32, 32)],
    "CATEGORY_WORD": [(48, 57), (65, 90), (95, 95), (97, 122)],
}


# ---- NFA -----------------------------------------------------------------------------------------------------------
class ByteNfa:
    def __init__(self):
        self.eps: List[List[int]] = []
        self.edges: List[List[Tuple[int, int, int]]] = []      # (byte lo, byte hi, target)

    def state(self) -> int:
        if len(self.eps) >= MAX_NFA_STATES:
            raise AutomatonError("pattern too large")
        self.eps.append([])
        self.edges.append([])
        return len(self.eps) - 1

    def chars(self, ranges: List[Tuple[int, int]]) -> Tuple[int, int]:
        """Fragment matching one code point out of ``ranges``."""
        s, t = self.state(), self.state()
        for lo, hi in _merge(ranges):
            for seq in utf8_sequences(lo, hi):
                cur = s
                for n, (blo, bhi) in enumerate(seq):
                    nxt = t if n == len(seq) - 1 else self.state()
                    self.edges[cur].append((blo, bhi, nxt))
                    cur = nxt
        return s, t


def _build(nfa: ByteNfa, items, dotall: bool) -> Tuple[int, int]:
    """Thompson construction over the parse tree of ``re``'s parser; returns (start, end) of the fragment."""
    import re._constants as C
    start = cur = nfa.state()
    for op, av in items:
        name = str(op)
        if name == "LITERAL":
            s, t = nfa.chars([(av, av)])
        elif name == "NOT_LITERAL":
            s, t = nfa.chars(_complement([(av, av)]))
        elif name == "ANY":
            s, t = nfa.chars([(0, MAX_CODEPOINT)] if dotall else _complement([(10, 10)]))
        elif name == "IN":
            neg, rs = False, []
            for iop, iav in av:
                iname = str(iop)
                if iname == "NEGATE":
                    neg = True
                elif iname == "LITERAL":
                    rs.append((iav, iav))
                elif iname == "RANGE":
                    rs.append((iav[0], iav[1]))
                elif iname == "CATEGORY":
                    cat = str(iav)
                    if cat.startswith("CATEGORY_NOT_"):
                        rs += _complement(_CATEGORIES["CATEGORY_" + cat[len("CATEGORY_NOT_"):]])
                    elif cat in _CATEGORIES:
                        rs += _CATEGORIES[cat]
                    else:
                        raise AutomatonError(f"character category {cat} is not supported")
                else:
                    raise AutomatonError(f"class item {iname} is not supported")
            s, t = nfa.chars(_complement(rs) if neg else rs)
        elif name == "BRANCH":
            s, t = nfa.state(), nfa.state()
            for alt in av[1]:
                a, b = _build(nfa, alt, dotall)
                nfa.eps[s].append(a)
                nfa.eps[b].append(t)
        elif name == "SUBPATTERN":
            s, t = _build(nfa, av[3], dotall)
        elif name in ("ATOMIC_GROUP",):
            s, t = _build(nfa, av, dotall)
        elif name in ("MAX_REPEAT", "MIN_REPEAT", "POSSESSIVE_REPEAT"):
            lo, hi, sub = av
            s = t = nfa.state()
            for _ in range(lo):
                a, b = _build(nfa, sub, dotall)
                nfa.eps[t].append(a)
                t = b
            if hi == C.MAXREPEAT:
                a, b = _build(nfa, sub, dotall)
                loop = nfa.state()
                nfa.eps[t].append(loop)
                nfa.eps[loop].append(a)
                nfa.eps[b].append(loop)
                t = loop
            else:
                end = nfa.state()
                for _ in range(hi - lo):
                    a, b = _build(nfa, sub, dotall)
                    nfa.eps[t].append(a)
                    nfa.eps[t].append(end)
                    t = b
                nfa.eps[t].append(end)
                t = end
        elif name == "AT":
            if str(av) in ("AT_BEGINNING", "AT_BEGINNING_STRING", "AT_END", "AT_END_STRING"):
                continue                                # the whole output is matched: edge anchors add nothing
            raise AutomatonError(f"anchor {av} is not supported")
        else:
            raise AutomatonError(f"regex construct {name} has no finite automaton here")
        nfa.eps[cur].append(s)
        cur = t
    return start, cur


def regex_to_nfa(pattern: str, dotall: bool = True) -> Tuple[ByteNfa, int, int]:
    import re
    try:
        import re._parser as parser
    except ImportError:                                 # pragma: no cover - older interpreters
        import sre_parse as parser
    try:
        tree = parser.parse(pattern)
    except (re.error, RecursionError, OverflowError) as e:
        raise AutomatonError(f"bad regex: {e}") from None
    if tree.state.flags & re.IGNORECASE:
        raise AutomatonError("case-insensitive patterns are not supported")
    nfa = ByteNfa()
    try:
        s, t = _build(nfa, list(tree), dotall or bool(tree.state.flags & re.DOTALL))
    except RecursionError:
        raise AutomatonError("pattern nests too deeply") from None
    return nfa, s, t


# ---- DFA -----------------------------------------------------------------------------------------------------------
class ByteDfa:
    """Dense DFA: ``table[state, byte]`` is the next state or -1 (dead); state 0 is the start."""

    def __init__(self, table: np.ndarray, accepting: np.ndarray):
        self.table, self.accepting = table, accepting

    @property
    def n_states(self) -> int:
        return self.table.shape[0]

    def step(self, state: int, byte: int) -> int:
        return int(self.table[state, byte]) if state >= 0 else -1

    def run(self, state: int, data: bytes) -> int:
        t = self.table
        for b in data:
            if state < 0:
                return -1
            state = int(t[state, b])
        return state

    @staticmethod
    def from_regex(pattern: str, dotall: bool = True) -> "ByteDfa":
        nfa, s, t = regex_to_nfa(pattern, dotall)
        return ByteDfa.from_nfa(nfa, s, t)

    @staticmethod
    def from_literals(choices: Sequence[bytes]) -> "ByteDfa":
        """The DFA of a fixed set of byte strings (a trie): ``guided_choice``."""
        nodes: List[Dict[int, int]] = [{}]
        acc = [False]
        for c in choices:
            cur = 0
            for b in c:
                nxt = nodes[cur].get(b)
                if nxt is None:
                    nodes.append({})
                    acc.append(False)
                    nxt = nodes[cur][b] = len(nodes) - 1
                cur = nxt
            acc[cur] = True
        table = np.full((len(nodes), 256), -1, np.int32)
        for i, n in enumerate(nodes):
            for b, j in n.items():
                table[i, b] = j
        return ByteDfa(table, np.asarray(acc, bool))

    @staticmethod
    def from_nfa(nfa: ByteNfa, start: int, accept: int) -> "ByteDfa":
        n = len(nfa.eps)
        # byte equivalence classes: bytes between two consecutive range boundaries behave alike everywhere
        cuts = {0, 256}
        for es in nfa.edges:
            for lo, hi, _ in es:
                cuts.add(lo)
                cuts.add(hi + 1)
        bounds = sorted(cuts)
        reps = bounds[:-1]

        def closure(seed) -> frozenset:
            seen, stack = set(seed), list(seed)
            while stack:
                for j in nfa.eps[stack.pop()]:
                    if j not in seen:
                        seen.add(j)
                        stack.append(j)
            return frozenset(seen)

        start_set = closure([start])
        ids = {start_set: 0}
        sets = [start_set]
        rows: List[List[int]] = []
        k = 0
        work = 0
        while k < len(sets):
            cur = sets[k]
            row = []
            edges = [e for s in cur for e in nfa.edges[s]]
            work += (len(edges) + len(cur)) * len(reps)
            if work > MAX_DFA_WORK:
                raise AutomatonError("the pattern's automaton is too expensive to build")
            for rb in reps:
                tgt = {t for lo, hi, t in edges if lo <= rb <= hi}
                if not tgt:
                    row.append(-1)
                    continue
                c = closure(tgt)
                j = ids.get(c)
                if j is None:
                    if len(sets) >= MAX_DFA_STATES:
                        raise AutomatonError("the pattern's automaton is too large")
                    j = ids[c] = len(sets)
                    sets.append(c)
                row.append(j)
            rows.append(row)
            k += 1
        S = len(sets)
        acc = np.array([accept in s for s in sets], bool)
        cls = np.asarray(rows, np.int32).reshape(S, len(reps))
        # states that cannot reach an accepting state are dead: "not dead" == "still a prefix of a full match"
        live = acc.copy()
        changed = True
        while changed:
            nxt = live.copy()
            ok = np.where(cls >= 0, live[np.clip(cls, 0, None)], False).any(axis=1)
            nxt |= ok
            changed = bool((nxt != live).any())
            live = nxt
        cls = np.where((cls >= 0) & live[np.clip(cls, 0, None)], cls, -1)
        if not live[0]:
            raise AutomatonError("the pattern matches nothing")
        width = np.diff(np.asarray(bounds))
        table = np.repeat(cls, width, axis=1).astype(np.int32)
        return ByteDfa(np.ascontiguousarray(table), acc)


# ---- token trie ----------------------------------------------------------------------------------------------------
class TokenTrie:
    """Trie of the vocabulary's token bytes.  Node 0 is the root; children of a node are contiguous in ``child_byte`` /
    ``child_node``; ``tok_start[n]:tok_start[n + 1]`` indexes the tokens that end at node ``n``."""

    def __init__(self, token_bytes: Sequence[bytes]):
        self.n_tokens = len(token_bytes)
        order = sorted((b, i) for i, b in enumerate(token_bytes) if b)
        children: List[Dict[int, int]] = [{}]
        ends: List[List[int]] = [[]]
        for b, i in order:
            cur = 0
            for byte in b:
                nxt = children[cur].get(byte)
                if nxt is None:
                    children.append({})
                    ends.append([])
                    nxt = children[cur][byte] = len(children) - 1
                cur = nxt
            ends[cur].append(i)
        N = len(children)
        self.child_start = np.zeros(N + 1, np.int32)
        cb, cn = [], []
        for n in range(N):
            self.child_start[n] = len(cb)
            for byte, node in sorted(children[n].items()):
                cb.append(byte)
                cn.append(node)
        self.child_start[N] = len(cb)
        self.child_byte = np.asarray(cb, np.uint8)
        self.child_node = np.asarray(cn, np.int32)
        self.tok_start = np.zeros(N + 1, np.int32)
        toks = []
        for n in range(N):
            self.tok_start[n] = len(toks)
            toks += ends[n]
        self.tok_start[N] = len(toks)
        self.tokens = np.asarray(toks, np.int32)
        self.n_nodes = N

    def walk_dfa(self, dfa: ByteDfa, state: int) -> np.ndarray:
        """Boolean mask over the vocabulary: tokens whose bytes keep ``dfa`` alive from ``state``."""
        out = np.zeros(self.n_tokens, bool)
        lib = _host_walk()
        if lib is not None:
            lib(self.child_start.ctypes.data, self.child_byte.ctypes.data, self.child_node.ctypes.data,
                self.tok_start.ctypes.data, self.tokens.ctypes.data, self.n_nodes, dfa.table.ctypes.data, dfa.n_states,
                state, out.ctypes.data)
            return out
        table = dfa.table
        stack = [(0, state)]
        cs, cb, cn, ts, tk = self.child_start, self.child_byte, self.child_node, self.tok_start, self.tokens
        while stack:
            node, st = stack.pop()
            for e in range(cs[node], cs[node + 1]):
                ns = table[st, cb[e]]
                if ns < 0:
                    continue
                ch = cn[e]
                if ts[ch] != ts[ch + 1]:
                    out[tk[ts[ch]:ts[ch + 1]]] = True
                stack.append((ch, ns))
        return out

    def walk(self, state, step) -> np.ndarray:
        """The same walk for any automaton given as ``step(state, byte) -> state or None``."""
        out = np.zeros(self.n_tokens, bool)
        stack = [(0, state)]
        cs, cb, cn, ts, tk = self.child_start, self.child_byte, self.child_node, self.tok_start, self.tokens
        while stack:
            node, st = stack.pop()
            for e in range(cs[node], cs[node + 1]):
                ns = step(st, int(cb[e]))
                if ns is None:
                    continue
                ch = cn[e]
                if ts[ch] != ts[ch + 1]:
                    out[tk[ts[ch]:ts[ch + 1]]] = True
                stack.append((ch, ns))
        return out


_walk_fn = False


def _host_walk():
    """The C++ trie walk of the host library, or None when the library is not built."""
    global _walk_fn
    if _walk_fn is False:
        try:
            from ..ops._lib import host
            f = host().poot_guided_walk_dfa
            P = ctypes.c_void_p
            f.argtypes = [P, P, P, P, P, ctypes.c_int, P, ctypes.c_int, ctypes.c_int, P]
            f.restype = None
            _walk_fn = f
        except Exception:
            _walk_fn = None
    return _walk_fn


class StateMasks:
    """Allowed-token masks by automaton state, computed on the first visit; bounded (cleared past a cap)."""

    def __init__(self):
        self.by_state: Dict[object, np.ndarray] = {}
        self.walks = 0                      # trie walks done: grows on a miss only

    def get(self, key, compute) -> np.ndarray:
        m = self.by_state.get(key)
        if m is None:
            if len(self.by_state) >= STATE_MASK_CAP:
                self.by_state.clear()
            m = self.by_state[key] = compute()
            self.walks += 1
        return m
