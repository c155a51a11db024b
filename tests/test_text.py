"""Text layer: tokenizers, streaming detokenisation, chat templates, guided decoding, tool calls (incl. hostile inputs)."""
import json

import numpy as np
import pytest

from poot_b200.text import chat, guided, tools
from poot_b200.text.codec import ByteTokenizer, GgufTokenizer, StreamDecoder


def test_byte_tokenizer_round_trip_and_streaming_never_splits_a_character():
    tk = ByteTokenizer(300)
    ids = tk.encode("héllo ✓", add_bos=False)
    assert tk.decode(ids) == "héllo ✓"
    sd = StreamDecoder(tk)
    pieces = [sd.push(i) for i in ids]
    assert "".join(pieces) + sd.flush() == "héllo ✓"
    assert all(p.encode("utf-8").decode("utf-8") == p for p in pieces)


def test_gguf_spm_and_bpe_tokenizers():
    spm = GgufTokenizer({"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": ["<unk>", "<s>", "</s>", "▁", "h", "e", "l", "o",
                                                                                    "▁he", "ll", "▁hell", "▁hello", "▁h"] + [f"<0x{b:02X}>" for b in range(256)],
                         "tokenizer.ggml.scores": [0, 0, 0, -1, -2, -2, -2, -2, -0.5, -0.6, -0.4, -0.1, -0.7] + [0.0] * 256,
                         "tokenizer.ggml.token_type": [2, 3, 3] + [1] * 10 + [6] * 256, "tokenizer.ggml.bos_token_id": 1})
    ids = spm.encode("hello")
    assert ids == [1, 11] and spm.decode(ids[1:]) == "hello"
    assert spm.decode(spm.encode("hé", add_bos=False)) == "hé"      # byte fallback
    enc = {b: c for b, c in __import__("poot_b200.text.codec", fromlist=["x"])._gpt2_byte_table().items()}
    toks = [enc[b] for b in range(256)] + ["he", "ll", "hell", "hello", "Ġw"]
    bpe = GgufTokenizer({"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": toks,
                         "tokenizer.ggml.merges": ["h e", "l l", "he ll", "hell o", "Ġ w"]})
    ids = bpe.encode("hello w", add_bos=False)
    assert [toks[i] for i in ids] == ["hello", "Ġw"] and bpe.decode(ids) == "hello w"


def test_chat_templates_render_and_refuse_hostile_templates():
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    out = chat.render_chat(msgs, family="qwen3")
    assert out.endswith("<|im_start|>assistant\n") and "<|im_start|>user\nhi<|im_end|>" in out
    assert "[INST] hi [/INST]" in chat.render_chat(msgs[1:], family="mistral", bos_token="<s>")
    custom = "{% for m in messages %}{{ m['role'] }}:{{ m['content'] }};{% endfor %}"
    assert chat.render_chat(msgs, template=custom) == "system:be brief;user:hi;"
    with pytest.raises(chat.TemplateError):
        chat.render_chat(msgs, template="{{ ''.__class__.__mro__ }}")           # sandbox escape attempt
    with pytest.raises(chat.TemplateError):
        chat.render_chat(msgs, template="{{ raise_exception('no system role') }}")
    with pytest.raises(chat.TemplateError):
        chat.render_chat(msgs, template="{% for i in range(3000) %}" + "x" * 2000 + "{% endfor %}")
    with pytest.raises(chat.TemplateError):
        chat.render_chat([{"content": "x"}])


@pytest.mark.parametrize("text,ok,complete", [
    ('{"a": [1, 2.5e3, true, null], "b": {"c": "x\\n"}}', True, True), ('{"a": [1, 2', True, False), ('{"a" 1}', False, False),
    ("[1,]", False, False), ('"unterminated', True, False), ("tru", True, False), ("truth", False, False), ("-0.5", True, True),
    ("01", False, False), ("[" * 100, False, False)])
def test_json_prefix_acceptor(text, ok, complete):
    c = guided.build_constraint({"json": True}, ByteTokenizer(300, eos=2), eos_token=2)
    assert c.feed_bytes(text.encode()) == ok
    if ok:
        assert c.m.complete(c.state) == complete


def test_schema_regex_and_choice_and_regex_constraints():
    import regex
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                               "tags": {"type": "array", "items": {"enum": ["a", "b"]}}},
              "required": ["name", "age"]}
    rx = regex.compile(guided.schema_to_regex(schema))
    assert rx.fullmatch('{"name": "bo", "age": 3, "tags": ["a", "b"]}') and rx.fullmatch('{"name":"x","age":-1}')
    assert not rx.fullmatch('{"name": "bo"}') and not rx.fullmatch('{"name": "bo", "age": 1.5}')
    tk = ByteTokenizer(300, eos=2)
    c = guided.build_constraint({"choice": ["yes", "no"]}, tk, eos_token=2)
    m = c.mask(300)
    allowed = {i for i in range(300) if m[i] == 0}
    assert allowed == {ord("y") + 3, ord("n") + 3}
    for ch in "no":
        c.advance(ord(ch) + 3)
    m = c.mask(300)
    assert {i for i in range(300) if m[i] == 0} == {2} and c.done()
    r = guided.build_constraint({"regex": r"[0-9]{3}-[a-z]+"}, tk, eos_token=2)
    for ch in "12":
        r.advance(ord(ch) + 3)
    m = r.mask(300)
    assert all((m[ord(d) + 3] == 0) for d in "0123456789") and m[ord("-") + 3] != 0
    with pytest.raises(guided.ConstraintError):
        guided.build_constraint({"regex": "(" * 5}, tk)
    with pytest.raises(guided.ConstraintError):
        guided.build_constraint({"regex": "a" * 100000}, tk)


def test_gbnf_grammar_machine():
    g = guided.Gbnf('root ::= "(" expr ")" | num\nexpr ::= num (op num)*\nnum ::= [0-9]+\nop ::= [+*-]\n')
    a = guided.GbnfAcceptor(g)
    assert a.clone().feed("(12+3*4)") and a.clone().feed("7")
    b = a.clone(); b.feed("(12+3)")
    assert b.complete()
    c = a.clone(); c.feed("(12+")
    assert not c.complete() and not c.clone().feed(")") and c.clone().feed("5")
    assert not a.clone().feed("x")
    with pytest.raises(guided.ConstraintError):
        guided.Gbnf("root ::= missing")
    with pytest.raises(guided.ConstraintError):
        guided.Gbnf("expr ::= [0-9]")


def test_tool_call_codecs_and_forced_tool_schema():
    text = 'let me check <tool_call>{"name": "get_weather", "arguments": {"city": "Oslo"}}</tool_call>'
    rest, calls = tools.parse_tool_calls(text, "hermes")
    assert rest == "let me check" and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo"}
    _, calls = tools.parse_tool_calls('[TOOL_CALLS] [{"name": "f", "arguments": {"x": 1}}]', "mistral")
    assert calls[0]["function"]["name"] == "f"
    _, calls = tools.parse_tool_calls('{"name": "f", "parameters": {"x": 1}}', "llama")
    assert json.loads(calls[0]["function"]["arguments"]) == {"x": 1}
    rest, calls = tools.parse_tool_calls("<tool_call>{broken</tool_call>", "hermes")
    assert calls == []
    sch = tools.forced_tool_schema([{"type": "function", "function": {"name": "f", "parameters": {"type": "object",
                                    "properties": {"x": {"type": "integer"}}, "required": ["x"]}}}], "f")
    import regex
    assert regex.fullmatch(guided.schema_to_regex(sch), '{"name": "f", "arguments": {"x": 4}}')
