"""GLM-5.2 (glm-dsa) chat framing: ``[gMASK]<sop>`` then ``<|system|>`` / ``<|user|>`` / ``<|assistant|>`` /
``<|observation|>`` role markers, each followed by a newline and the text; ``<think>`` opens reasoning
(reference: src/encoding/glm_dsa.py:30-55 for the single-turn form)."""
from __future__ import annotations

import json
import re
from typing import Any

PREFIX = "[gMASK]<sop>"
DEFAULT_SYSTEM_PROMPT = "You are a helpful assistant."


def _text(content: Any) -> str:
    if isinstance(content, list):
        return "".join(p.get("text", "") for p in content if isinstance(p, dict))
    return content or ""


def render(messages: list[dict[str, Any]], tools=None, thinking: bool = False, add_generation_prompt: bool = True) -> str:
    out = PREFIX
    if tools:
        out += "<|system|>\n# Tools\n\nYou may call these functions; reply with <tool_call>{name}\n<arg_key>k</arg_key>\n" \
               "<arg_value>v</arg_value>\n</tool_call>.\n" + "\n".join(json.dumps(t.get("function", t), ensure_ascii=False) for t in tools)
    for m in messages:
        role = m.get("role")
        if role == "system":
            out += "<|system|>\n" + _text(m.get("content"))
        elif role in ("user", "developer"):
            out += "<|user|>\n" + _text(m.get("content"))
        elif role == "tool":
            out += "<|observation|>\n" + _text(m.get("content"))
        elif role == "assistant":
            out += "<|assistant|>"
            rc = m.get("reasoning_content")
            out += "\n<think>" + rc + "</think>" if rc else "\n<think></think>"
            out += "\n" + _text(m.get("content")) if m.get("content") else ""
            for tc in m.get("tool_calls") or []:
                fn = tc.get("function", tc)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except Exception:
                        args = {"arguments": args}
                out += "\n<tool_call>" + fn.get("name", "")
                for k, v in args.items():
                    out += f"\n<arg_key>{k}</arg_key>\n<arg_value>{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}</arg_value>"
                out += "\n</tool_call>"
        else:
            raise ValueError(f"unknown role {role!r}")
    if add_generation_prompt:
        out += "<|assistant|>"
        out += "\n<think>" if thinking else "\n<think></think>\n"
    return out


_TOOL = re.compile(r"<tool_call>(?P<name>[^\n<]*)(?P<body>.*?)</tool_call>", re.S)
_ARG = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)


def parse_completion(text: str) -> dict[str, Any]:
    reasoning = None
    if "</think>" in text:
        head, text = text.split("</think>", 1)
        reasoning = head.replace("<think>", "").strip() or None
    calls = []
    for i, m in enumerate(_TOOL.finditer(text)):
        args = {}
        for k, v in _ARG.findall(m.group("body")):
            try:
                args[k.strip()] = json.loads(v)
            except Exception:
                args[k.strip()] = v
        calls.append({"id": f"call_{i}", "type": "function",
                      "function": {"name": m.group("name").strip(), "arguments": json.dumps(args, ensure_ascii=False)}})
    content = _TOOL.sub("", text).strip()
    return {"role": "assistant", "content": content, "reasoning_content": reasoning, "tool_calls": calls or None}
