"""Chat templates: the checkpoint's Jinja template rendered in a sandbox with budgets, or a named fallback format.

The reference renders ``chat_template`` with minijinja under output / iteration budgets and falls back to a small
set of built-in ``ChatFormat``s when a checkpoint ships none (crates/poot-text/src/lib.rs:19-33).
"""
from __future__ import annotations

from typing import Dict, List, Optional

MAX_RENDERED = 4 * 1024 * 1024


class TemplateError(ValueError):
    pass


FALLBACKS: Dict[str, str] = {
    "chatml": "{% for m in messages %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n{% endfor %}"
              "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}",
    "llama3": "{{ bos_token }}{% for m in messages %}<|start_header_id|>{{ m.role }}<|end_header_id|>\n\n"
              "{{ m.content }}<|eot_id|>{% endfor %}{% if add_generation_prompt %}<|start_header_id|>assistant"
              "<|end_header_id|>\n\n{% endif %}",
    "mistral": "{{ bos_token }}{% for m in messages %}{% if m.role == 'user' %}[INST] {{ m.content }} [/INST]"
               "{% elif m.role == 'assistant' %}{{ m.content }}{{ eos_token }}{% endif %}{% endfor %}",
    "plain": "{% for m in messages %}{{ m.content }}\n{% endfor %}",
}
FAMILY_DEFAULT = {"llama": "llama3", "mistral": "mistral", "mixtral": "mistral", "qwen2": "chatml", "qwen3": "chatml",
                  "qwen3moe": "chatml", "smollm3": "chatml", "olmo2": "chatml", "phi3": "chatml", "granite": "chatml"}


def render_chat(messages: List[dict], template: Optional[str] = None, family: str = "llama",
                add_generation_prompt: bool = True, bos_token: str = "", eos_token: str = "",
                tools: Optional[list] = None, keep_parts: bool = False) -> str:
    """``keep_parts`` hands list-valued message contents to the template as they are (multimodal templates walk the
    parts and write a placeholder per image); otherwise a list collapses to the concatenation of its text parts."""
    from jinja2 import TemplateError as JTE
    from jinja2.sandbox import ImmutableSandboxedEnvironment
    for m in messages:
        if not isinstance(m, dict) or "role" not in m:
            raise TemplateError("every message needs a role")
        if not isinstance(m.get("content", ""), (str, list)) and m.get("content") is not None:
            raise TemplateError("message content must be text or a list of parts")
    src = template or FALLBACKS[FAMILY_DEFAULT.get(family, "chatml")]
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)

    def raise_exception(msg):
        raise TemplateError(str(msg))
    env.globals["raise_exception"] = raise_exception
    norm = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list) and not keep_parts:
            c = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") == "text")
        norm.append({**m, "content": c if (keep_parts and isinstance(c, list)) else (c or "")})
    try:
        out = env.from_string(src).render(messages=norm, add_generation_prompt=add_generation_prompt,
                                          bos_token=bos_token, eos_token=eos_token, tools=tools)
    except JTE as e:
        raise TemplateError(f"chat template failed: {e}") from None
    if len(out) > MAX_RENDERED:
        raise TemplateError("rendered prompt exceeds the output budget")
    return out
