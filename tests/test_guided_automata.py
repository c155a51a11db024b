"""Guided decoding automata: regex -> byte DFA (checked against the ``regex`` module on random strings), UTF-8 classes,
tokens that hold part of a character, per-state cached masks, JSON and GBNF machines over bytes."""
import random

import numpy as np
import pytest

from poot_b200.text import guided
from poot_b200.text.automata import AutomatonError, ByteDfa, StateMasks, TokenTrie, utf8_sequences
from poot_b200.text.codec import ByteTokenizer


def _accepts(dfa, data: bytes):
    st = dfa.run(0, data)
    return st >= 0, (st >= 0 and bool(dfa.accepting[st]))


PATTERNS = [r"[0-9]{3}-[a-z]+", r"(?:ab|cd)*e?", r"\d+(\.\d+)?([eE][+-]?\d+)?", r'"([^"\\]|\\.)*"', r"a{2,4}b{0,2}c",
            r"(yes|no|maybe)", r"[^\x00-\x1f]{1,5}", r"\w+@\w+\.(com|org)", r"é+|ü{2}", r".{0,3}x", r"\s*[A-Z][a-z]*\s*"]


@pytest.mark.parametrize("pattern", PATTERNS)
def test_dfa_agrees_with_the_regex_module_on_prefixes_and_full_matches(pattern):
    import regex
    rx = regex.compile(pattern, flags=regex.DOTALL | regex.ASCII)     # \d \w \s are the ASCII classes here
    dfa = ByteDfa.from_regex(pattern)
    rng = random.Random(hash(pattern) & 0xFFFF)
    alphabet = 'abcdexyz019-.eE+"\\ \n@comrgyesnmb_éü\x01AZ'
    for _ in range(400):
        s = "".join(rng.choice(alphabet) for _ in range(rng.randrange(0, 9)))
        alive, full = _accepts(dfa, s.encode("utf-8"))
        assert alive == (rx.fullmatch(s, partial=True) is not None), (pattern, s)
        assert full == (rx.fullmatch(s) is not None), (pattern, s)


def test_utf8_sequences_cover_exactly_their_code_points():
    for lo, hi in ((0, 0x10FFFF), (0x80, 0x7FF), (0x7F0, 0x810), (0xD700, 0xE100), (0xFFF0, 0x10010), (0x4E00, 0x4E3F)):
        seqs = list(utf8_sequences(lo, hi))
        rng = random.Random(lo)
        for cp in [lo, hi] + [rng.randrange(0, 0x110000) for _ in range(300)]:
            if 0xD800 <= cp <= 0xDFFF:
                continue
            b = chr(cp).encode("utf-8")
            hit = any(len(q) == len(b) and all(a <= x <= c for x, (a, c) in zip(b, q)) for q in seqs)
            assert hit == (lo <= cp <= hi), (hex(lo), hex(hi), hex(cp))


def test_unsupported_constructs_and_oversized_patterns_are_refused():
    for bad in (r"(a)\1", r"(?=a)b", r"(?i)abc", r"\bword"):
        with pytest.raises(AutomatonError):
            ByteDfa.from_regex(bad)
    with pytest.raises(AutomatonError):
        ByteDfa.from_regex("(a{1,60}){1,60}b{1,60}" * 8)            # state bound
    tk = ByteTokenizer(300, eos=2)
    with pytest.raises(guided.ConstraintError):
        guided.build_constraint({"regex": r"(?=a)b"}, tk)


class _Tok:
    """A tokenizer over an explicit byte table (tokens may split UTF-8 characters, as byte-level BPE vocabularies do)."""

    def __init__(self, table):
        self.table = table

    def vocab_size(self):
        return len(self.table)

    def token_bytes(self, t):
        return self.table[t]


def test_tokens_that_split_a_character_are_allowed_exactly_when_the_bytes_fit():
    e_acute = "é".encode()          # c3 a9
    han = "中".encode()              # e4 b8 ad
    table = [b"", b"a", e_acute, e_acute[:1], e_acute[1:], han, han[:2], han[2:], han[:1], b"\xff", b"ab", "é中".encode()]
    tk = _Tok(table)
    c = guided.build_constraint({"regex": "[é中]+a"}, tk)
    allowed = {i for i, v in enumerate(c.mask(len(table))) if v == 0}
    assert allowed == {2, 3, 5, 6, 8, 11}          # whole characters and their proper byte prefixes; not 'a', not stray bytes
    c.advance(3)                                     # first byte of é
    assert {i for i, v in enumerate(c.mask(len(table))) if v == 0} == {4}       # only its continuation byte
    c.advance(4)
    assert {i for i, v in enumerate(c.mask(len(table))) if v == 0} == {1, 2, 3, 5, 6, 8, 11}
    c.advance(1)
    assert c.done()


def test_masks_are_computed_once_per_state_and_shared_between_requests():
    tk = ByteTokenizer(300, eos=2)
    a = guided.build_constraint({"regex": r"(ab)*c"}, tk, eos_token=2)
    b = guided.build_constraint({"regex": r"(ab)*c"}, tk, eos_token=2)
    assert a.masks is b.masks and a.m is b.m         # one automaton and one mask cache per (pattern, tokenizer)
    walks0 = a.masks.walks
    for _ in range(6):                               # the loop revisits two states
        a.mask(300); a.advance(ord("a") + 3)
        a.mask(300); a.advance(ord("b") + 3)
    assert a.masks.walks - walks0 <= 3
    b.mask(300)                                      # the other request starts in a state that is cached already
    assert a.masks.walks - walks0 <= 3
    m = a.mask(300)
    assert m[ord("c") + 3] == 0 and m[ord("a") + 3] == 0 and m[ord("b") + 3] != 0 and m[2] != 0
    a.advance(ord("c") + 3)
    assert a.mask(300)[2] == 0 and a.done()


def test_trie_walk_in_the_host_library_equals_the_python_walk():
    rng = random.Random(5)
    toks = [bytes(rng.choice(b"abc019-.") for _ in range(rng.randrange(1, 6))) for _ in range(2000)] + [b""]
    trie = TokenTrie(toks)
    dfa = ByteDfa.from_regex(r"[0-9]{3}-[a-c]+\.?")
    for state in range(dfa.n_states):
        fast = trie.walk_dfa(dfa, state)
        slow = trie.walk(state, lambda s, b: (None if dfa.table[s, b] < 0 else int(dfa.table[s, b])))
        brute = np.array([bool(t) and dfa.run(state, t) >= 0 for t in toks])
        assert np.array_equal(fast, slow) and np.array_equal(fast, brute)


def test_json_and_grammar_machines_step_over_bytes():
    tk = ByteTokenizer(300, eos=2)
    j = guided.build_constraint({"json": True}, tk, eos_token=2)
    assert j.feed_bytes('{"a": [1, 2.5e3, true, null], "b": {"c": "x\\n é"}}'.encode())
    assert j.m.complete(j.state) and j.mask(300)[2] == 0
    for bad in (b'{"a" 1}', b"[1,]", b"01", b"truth"):
        assert not guided.build_constraint({"json": True}, tk).feed_bytes(bad)
    p = guided.build_constraint({"json": True}, tk, eos_token=2)
    assert p.feed_bytes(b'{"k": "caf\xc3')           # the middle of a two-byte character inside a string
    m = p.mask(300)
    assert m[0xA9 + 3] == 0 and m[ord("a") + 3] != 0 and m[2] != 0
    g = guided.build_constraint({"grammar": 'root ::= "(" expr ")" | num\nexpr ::= num (op num)*\nnum ::= [0-9]+\nop ::= [+*-]\n'},
                                tk, eos_token=2)
    assert g.feed_bytes(b"(12+3")
    m = g.mask(300)
    assert {chr(i - 3) for i in range(3, 259) if m[i] == 0} == set("0123456789+*-)")
    assert g.feed_bytes(b")") and g.done()


def test_schema_constraint_through_the_driver_interface():
    tk = ByteTokenizer(300, eos=2)
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "n": {"type": "integer"}}, "required": ["name", "n"]}
    c = guided.build_constraint({"json_schema": schema}, tk, eos_token=2)
    text = '{"name": "bo", "n": 42}'
    for ch in text.encode():
        assert c.mask(300)[ch + 3] == 0, chr(ch)
        c.advance(ch + 3)
    assert c.mask(300)[2] == 0
    d = c.clone()
    assert d.state == c.state and d.masks is c.masks
