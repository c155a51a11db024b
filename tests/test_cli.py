"""``generate`` flags: strict parsing, one-shot, reverse prompts, conversation mode (host engine)."""
import io

import pytest

from poot_b200.cli.__main__ import main
from poot_b200.cli.generate import parse_generate, run_generate
from poot_b200.llm import LLM


def test_defaults_match_the_llama_cli_subset():
    a = parse_generate(["-m", "x.gguf", "-p", "hi"])
    assert (a.predict, a.ctx_size, a.temp, a.top_k, a.top_p, a.min_p, a.repeat_penalty) == (-1, 0, 0.0, 40, 0.95, 0.05, 1.0)
    assert a.show_timings and not a.ignore_eos and a.backend == "auto" and a.seed is None
    a = parse_generate(["-m", "x", "-f", "p.txt", "-n", "7", "-c", "2048", "--temp", "0.7", "-s", "3", "-r", "A", "-r", "B",
                        "--no-show-timings", "--ignore-eos"])
    assert a.predict == 7 and a.ctx_size == 2048 and a.reverse_prompt == ["A", "B"] and not a.show_timings and a.seed == 3


@pytest.mark.parametrize("argv", [
    ["-p", "hi"],                                       # no model
    ["-m", "x"],                                        # no prompt
    ["-m", "x", "-p", "a", "-f", "b"],
    ["-m", "x", "-p", "a", "--bogus"],
    ["-m", "x", "-p", "a", "-n", "0"],
    ["-m", "x", "-p", "a", "--top-p", "2"],
    ["-m", "x", "-p", "a", "--no-chat-template", "--system-prompt", "s"],
    ["-m", "x", "-p", "a", "--backend", "vulkan"],
    ["-m", "x", "-p", "a", "--temp", "abc"],
])
def test_strict_parsing_refuses(argv):
    with pytest.raises(ValueError):
        parse_generate(argv)
    assert main(["generate", *argv]) == 2


def test_one_shot_raw_prompt_on_the_host_engine():
    a = parse_generate(["-m", "fake", "--no-chat-template", "-p", "xa", "-n", "5", "--no-show-timings"])
    out = io.StringIO()
    t = run_generate(a, llm=LLM.fake(), out=out)
    assert out.getvalue() == "bcdef\n" and t["generated"] == 5 and t["prompt_tokens"] == 3


def test_reverse_prompt_stops_and_is_not_printed():
    a = parse_generate(["-m", "fake", "--no-chat-template", "-p", "a", "-n", "20", "-r", "ef", "--no-show-timings"])
    out = io.StringIO()
    run_generate(a, llm=LLM.fake(), out=out)
    assert out.getvalue() == "bcd\n"


def test_conversation_keeps_the_sequence_and_feeds_only_new_turns():
    llm = LLM.fake(max_seq=2048, num_blocks=256)
    a = parse_generate(["-m", "fake", "--conversation", "-p", "first", "-n", "4", "--no-show-timings"])
    out = io.StringIO()
    t = run_generate(a, llm=llm, out=out, inp=io.StringIO("second\n\n"))
    steps = llm.driver.engine.steps
    fed = sum(len(s.tokens) for s in steps)
    assert t["generated"] == 8                      # two turns of four tokens
    assert fed < 2 * t["prompt_tokens"]             # the first turn was not fed again
    assert not llm.driver.seqs                      # released at the end


def test_commands():
    assert main([]) == 2 and main(["--help"]) == 0
    assert main(["caption", "-m", "x"]) == 2 and main(["embed", "-m", "x"]) == 2 and main(["nope"]) == 2
    assert main(["generate", "-m", "fake", "--no-chat-template", "-p", "a", "-n", "2", "--no-show-timings"]) == 0


def test_plan_command_reports_the_compiled_step(tmp_path, capsys):
    """``poot plan`` compiles one step from the checkpoint's header alone and prints census, digest, numerics class,
    state commit and what the build says of each dispatched kernel; ``--json`` gives the same as one object."""
    import json
    from poot_b200.cli.__main__ import main
    from tests.test_families import header
    d = tmp_path / "ckpt"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({**header("qwen3next"), "model_type": "qwen3_next"}))
    assert main(["plan", str(d), "--tokens", "4", "--capacity", "32"]) == 0
    out = capsys.readouterr().out
    assert "qwen3next: 1 x 4 tokens" in out and "numerics narrowing" in out and "poot_gdn_scan" in out
    assert "state written in place: layers.1.k_pool" in out and "state copied after the step: layers.0.conv_state" in out
    assert main(["plan", str(d), "--json"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["family"] == "qwen3next" and rep["census"]["poot_gdn_scan"] == 2 and rep["numerics"]["tolerance"] == 5e-3
    assert rep["kernels"]["poot_gdn_scan"]["entry"] == "gdn_scan_kernel" and rep["kernels"]["poot_gdn_scan"]["spilling"] == []
    assert main(["plan", str(tmp_path / "missing")]) == 1
