"""Tool-call codecs: turn generated text into OpenAI ``tool_calls`` (Hermes, Llama-3 JSON, Mistral ``[TOOL_CALLS]``).

Counterpart of the reference's ``ToolCallCodec`` (crates/poot-text/src/lib.rs:19-33).
"""
from __future__ import annotations

import json
import re
import uuid
from typing import List, Optional, Tuple


def _call(name: str, args) -> dict:
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
            "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args)}}


def parse_tool_calls(text: str, style: str = "hermes") -> Tuple[str, List[dict]]:
    """Returns (remaining assistant text, tool calls)."""
    calls: List[dict] = []
    if style == "hermes":
        def grab(m):
            try:
                o = json.loads(m.group(1))
                calls.append(_call(o["name"], o.get("arguments", {})))
                return ""
            except (json.JSONDecodeError, KeyError, TypeError):
                return m.group(0)
        rest = re.sub(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", grab, text, flags=re.S)
        return rest.strip(), calls
    if style == "mistral":
        m = re.search(r"\[TOOL_CALLS\]\s*(\[.*\])", text, flags=re.S)
        if m:
            try:
                for o in json.loads(m.group(1)):
                    calls.append(_call(o["name"], o.get("arguments", {})))
                return text[:m.start()].strip(), calls
            except (json.JSONDecodeError, KeyError, TypeError):
                pass
        return text, calls
    if style == "llama":
        s = text.strip()
        if s.startswith("<|python_tag|>"):
            s = s[len("<|python_tag|>"):]
        try:
            o = json.loads(s)
            if isinstance(o, dict) and "name" in o:
                calls.append(_call(o["name"], o.get("parameters", o.get("arguments", {}))))
                return "", calls
        except json.JSONDecodeError:
            pass
        return text, calls
    raise ValueError(f"unknown tool-call style {style!r}")


def forced_tool_schema(tools: list, name: Optional[str] = None) -> dict:
    """JSON schema a forced tool call must satisfy (used as a guided-decoding constraint)."""
    fns = [t["function"] for t in tools if t.get("type") == "function"]
    if name is not None:
        fns = [f for f in fns if f["name"] == name]
    if not fns:
        raise ValueError("no matching tool")
    alts = [{"type": "object", "properties": {"name": {"const": f["name"]}, "arguments": f.get("parameters", {"type": "object"})},
             "required": ["name", "arguments"]} for f in fns]
    return alts[0] if len(alts) == 1 else {"anyOf": alts}
