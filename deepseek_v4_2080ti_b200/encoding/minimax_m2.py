"""MiniMax-M2 chat framing: ``]~!b[`` opens the conversation, every turn is ``]~b]<role>\\n<text>[e~[\\n`` with roles
``system`` / ``user`` / ``ai`` / ``tool``; ``<think>\\n`` opens reasoning
(reference: src/encoding/minimax_m2.py:30-57 for the single-turn form)."""
from __future__ import annotations

import json
from typing import Any

BOD = "]~!b["
BOS = "]~b]"
EOS = "[e~["
DEFAULT_SYSTEM_PROMPT = "You are a helpful assistant."


def _text(content: Any) -> str:
    if isinstance(content, list):
        return "".join(p.get("text", "") for p in content if isinstance(p, dict))
    return content or ""


def render(messages: list[dict[str, Any]], tools=None, thinking: bool = False, add_generation_prompt: bool = True) -> str:
    msgs = list(messages)
    system = DEFAULT_SYSTEM_PROMPT
    if msgs and msgs[0].get("role") == "system":
        system = _text(msgs.pop(0).get("content"))
    if tools:
        system += "\n\n# Tools\n" + "\n".join("<tool>" + json.dumps(t.get("function", t), ensure_ascii=False) + "</tool>" for t in tools)
    out = BOD + BOS + "system\n" + system + EOS + "\n"
    for m in msgs:
        role = m.get("role")
        name = {"user": "user", "developer": "user", "assistant": "ai", "tool": "tool", "system": "system"}.get(role)
        if name is None:
            raise ValueError(f"unknown role {role!r}")
        body = _text(m.get("content"))
        if role == "assistant":
            if m.get("reasoning_content"):
                body = "<think>\n" + m["reasoning_content"] + "\n</think>\n\n" + body
            for tc in m.get("tool_calls") or []:
                fn = tc.get("function", tc)
                body += "\n<minimax:tool_call>\n" + json.dumps({"name": fn.get("name"), "arguments": fn.get("arguments")},
                                                              ensure_ascii=False) + "\n</minimax:tool_call>"
        out += BOS + name + "\n" + body + EOS + "\n"
    if add_generation_prompt:
        out += BOS + "ai\n"
        if thinking:
            out += "<think>\n"
    return out
