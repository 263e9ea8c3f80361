"""Chat-completions request normalisation: content parts, tools, thinking mode, stop strings and
tool-call extraction.  Pure Python, no model or tokenizer dependency
(reference surface: pocketllm/protocol/chat.py:24-258)."""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence

from ..api.errors import ConfigurationError

_ROLES = {"system", "user", "assistant", "tool", "developer"}
_EFFORTS = {"low", "medium", "high", "max"}


def flatten_content(content: Any) -> str:
    """OpenAI message content (string, None, or a list of typed parts) -> plain text."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if isinstance(content, Mapping):
        content = [content]
    if not isinstance(content, Sequence):
        raise ConfigurationError("message content must be a string or a list of parts")
    pieces: list[str] = []
    for part in content:
        if isinstance(part, str):
            pieces.append(part)
            continue
        if not isinstance(part, Mapping):
            raise ConfigurationError("content parts must be objects")
        kind = part.get("type", "text")
        if kind in ("text", "input_text", "output_text"):
            pieces.append(str(part.get("text", "")))
        elif kind in ("image_url", "input_image", "input_audio", "file"):
            raise ConfigurationError(f"content part of type {kind!r} is not supported by a text-only model")
        else:
            raise ConfigurationError(f"unknown content part type {kind!r}")
    return "".join(pieces)


def normalise_tools(tools: Any) -> list[dict[str, Any]]:
    if not tools:
        return []
    if not isinstance(tools, Sequence) or isinstance(tools, (str, bytes)):
        raise ConfigurationError("tools must be a list")
    out = []
    for t in tools:
        if not isinstance(t, Mapping):
            raise ConfigurationError("each tool must be an object")
        fn = t.get("function", t)
        name = fn.get("name")
        if not name or not isinstance(name, str):
            raise ConfigurationError("each tool needs a function name")
        out.append({"type": "function", "function": {"name": name, "description": fn.get("description", ""),
                                                      "parameters": fn.get("parameters") or {"type": "object", "properties": {}}}})
    return out


def tool_choice_instruction(tool_choice: Any, tools: list[dict[str, Any]]) -> str:
    """Turn ``tool_choice`` into a sentence appended to the system prompt (models here have no native field for it)."""
    if not tools or tool_choice in (None, "auto"):
        return ""
    if tool_choice == "none":
        return "Do not call any tool; answer directly."
    if tool_choice == "required":
        return "You must call one of the available tools."
    if isinstance(tool_choice, Mapping):
        name = (tool_choice.get("function") or {}).get("name") or tool_choice.get("name")
        if not name or name not in {t["function"]["name"] for t in tools}:
            raise ConfigurationError("tool_choice names a tool that is not in tools")
        return f"You must call the tool named {name}."
    raise ConfigurationError("tool_choice must be 'auto', 'none', 'required' or a function selector")


def thinking_options(body: Mapping[str, Any]) -> tuple[bool, str | None]:
    """(thinking enabled, effort) from ``thinking`` / ``reasoning_effort`` / ``chat_template_kwargs``."""
    enabled = False
    effort = body.get("reasoning_effort")
    th = body.get("thinking")
    if isinstance(th, Mapping):
        enabled = th.get("type", "enabled") != "disabled"
    elif isinstance(th, bool):
        enabled = th
    kw = body.get("chat_template_kwargs") or {}
    if isinstance(kw, Mapping):
        if "enable_thinking" in kw:
            enabled = bool(kw["enable_thinking"])
        if "thinking" in kw:
            enabled = bool(kw["thinking"])
    if effort is not None:
        effort = str(effort).lower()
        if effort not in _EFFORTS and effort != "none":
            raise ConfigurationError(f"reasoning_effort must be one of {sorted(_EFFORTS)}")
        enabled = effort != "none"
        effort = None if effort == "none" else effort
    return enabled, effort


def truncate_at_stop(text: str, stops: Sequence[str]) -> tuple[str, bool]:
    """Cut ``text`` at the earliest stop string. Returns (text, hit)."""
    cut = None
    for s in stops:
        if not s:
            continue
        i = text.find(s)
        if i >= 0 and (cut is None or i < cut):
            cut = i
    return (text, False) if cut is None else (text[:cut], True)


def held_back_suffix(text: str, stops: Sequence[str]) -> int:
    """Number of trailing characters that could still grow into a stop string (held back while streaming)."""
    hold = 0
    for s in stops:
        for n in range(min(len(s) - 1, len(text)), 0, -1):
            if text.endswith(s[:n]):
                hold = max(hold, n)
                break
    return hold


_TOOL_BLOCK = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_THINK = re.compile(r"<think>(.*?)</think>", re.S)


def split_reasoning(text: str) -> tuple[str, str]:
    """(reasoning, answer): pulls a leading <think>…</think> block out of the completion."""
    m = _THINK.search(text)
    if m:
        return m.group(1).strip(), (text[:m.start()] + text[m.end():]).strip()
    if "</think>" in text:                      # template opened the block for the model
        head, tail = text.split("</think>", 1)
        return head.replace("<think>", "").strip(), tail.strip()
    return "", text


def extract_tool_calls(text: str) -> tuple[str, list[dict[str, Any]]]:
    """Find JSON tool calls in ``<tool_call>{…}</tool_call>`` blocks; returns (remaining text, OpenAI tool_calls)."""
    calls = []
    for m in _TOOL_BLOCK.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        name = obj.get("name")
        if not isinstance(name, str):
            continue
        args = obj.get("arguments", obj.get("parameters", {}))
        calls.append({"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function",
                      "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}})
    rest = _TOOL_BLOCK.sub("", text).strip() if calls else text
    return rest, calls


def fallback_prompt(messages: Sequence[Mapping[str, Any]], add_generation_prompt: bool = True) -> str:
    """Template-free rendering used when a checkpoint ships no chat template."""
    lines = [f"<|{m['role']}|>\n{m['content']}" for m in messages]
    if add_generation_prompt:
        lines.append("<|assistant|>\n")
    return "\n".join(lines)


def response_format_schema(response_format: Any) -> Any:
    """What a ``response_format`` asks the reply to follow: None for plain text, ``{"type": "object"}`` for
    ``json_object``, the schema itself for ``json_schema`` (``{"json_schema": {"schema": ...}}`` or the bare schema)."""
    if response_format is None:
        return None
    if not isinstance(response_format, Mapping):
        raise ConfigurationError("response_format must be an object")
    kind = response_format.get("type")
    if kind in (None, "text"):
        return None
    if kind == "json_object":
        return {"type": "object"}
    if kind == "json_schema":
        inner = response_format.get("json_schema")
        if not isinstance(inner, Mapping):
            raise ConfigurationError("response_format.json_schema must be an object")
        return inner.get("schema", inner)
    raise ConfigurationError(f"unknown response_format type {kind!r}")


def response_format_instruction(schema: Any) -> str:
    """The instruction a chat family without its own response-format block carries in the system message."""
    import json
    if schema == {"type": "object"}:
        return "Reply with one valid JSON object and nothing else."
    return ("Reply with one JSON value that strictly follows this JSON schema, and nothing else:\n"
            + json.dumps(schema, ensure_ascii=False))


@dataclass
class ChatRequest:
    messages: list[dict[str, Any]]
    tools: list[dict[str, Any]] = field(default_factory=list)
    tool_instruction: str = ""
    response_schema: Any = None
    thinking: bool = False
    reasoning_effort: str | None = None
    stream: bool = False
    model: str | None = None
    add_generation_prompt: bool = True

    @classmethod
    def from_body(cls, body: Mapping[str, Any]) -> "ChatRequest":
        if not isinstance(body, Mapping):
            raise ConfigurationError("request body must be a JSON object")
        raw = body.get("messages")
        if not isinstance(raw, Sequence) or isinstance(raw, (str, bytes)) or not raw:
            raise ConfigurationError("messages must be a non-empty list")
        msgs: list[dict[str, Any]] = []
        for m in raw:
            if not isinstance(m, Mapping):
                raise ConfigurationError("each message must be an object")
            role = m.get("role")
            if role not in _ROLES:
                raise ConfigurationError(f"unknown message role {role!r}")
            item: dict[str, Any] = {"role": "system" if role == "developer" else role,
                                    "content": flatten_content(m.get("content"))}
            if m.get("tool_calls"):
                item["tool_calls"] = list(m["tool_calls"])
            if m.get("tool_call_id"):
                item["tool_call_id"] = m["tool_call_id"]
            if m.get("name"):
                item["name"] = m["name"]
            msgs.append(item)
        tools = normalise_tools(body.get("tools"))
        thinking, effort = thinking_options(body)
        return cls(messages=msgs, tools=tools, tool_instruction=tool_choice_instruction(body.get("tool_choice"), tools),
                   thinking=thinking, reasoning_effort=effort, stream=bool(body.get("stream", False)),
                   model=body.get("model"), response_schema=response_format_schema(body.get("response_format")))

    def messages_with_instruction(self, native_response_format: bool = False) -> list[dict[str, Any]]:
        """The messages with the tool-choice instruction and the response format folded into the system message (one is
        added when the conversation has none).  ``native_response_format``: the chat family renders a
        ``response_format`` key of the system message itself (DeepSeek-V4); otherwise the schema travels as text."""
        extra = self.tool_instruction
        if self.response_schema is not None and not native_response_format:
            extra = (extra + "\n\n" + response_format_instruction(self.response_schema)).strip()
        if not extra and self.response_schema is None:
            return self.messages
        msgs = [dict(m) for m in self.messages]
        if not (msgs and msgs[0]["role"] == "system"):
            msgs.insert(0, {"role": "system", "content": ""})
        if extra:
            msgs[0]["content"] = (msgs[0]["content"] + "\n\n" + extra).strip()
        if self.response_schema is not None and native_response_format:
            msgs[0]["response_format"] = self.response_schema
        return msgs
