"""DeepSeek-V4 chat encoding.

Format (reference: src/encoding/deepseek_v4.py:16-118, render rules :242-420, tool merging :425-527):
* the conversation opens with the BOS token; a system message is emitted as plain text, followed by the tool
  catalogue when tools are offered;
* a user turn is ``<｜User｜>`` + text; tool results have no role of their own, they become
  ``<tool_result>..</tool_result>`` blocks of a user turn (consecutive tool results share one turn, ordered like the
  calls that produced them);
* an assistant turn is ``<｜Assistant｜>`` then ``<think>`` + reasoning + ``</think>`` in thinking mode (only for turns
  after the last user message, unless tools are in play) or a bare ``</think>`` in chat mode, then the text, then the
  tool calls as a ``<｜DSML｜tool_calls>`` block, then the EOS token;
* in thinking mode a "high" / "max" reasoning-effort preamble is put in front of the first message.
"""
from __future__ import annotations

import copy
import json
import re
from typing import Any

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML = "｜DSML｜"
USER, ASSISTANT = "<｜User｜>", "<｜Assistant｜>"
LATEST_REMINDER = "<｜latest_reminder｜>"
# quick-instruction tasks: a task token after the message asks for a classification-style answer
TASK_TOKENS = {"action": "<｜action｜>", "query": "<｜query｜>", "authority": "<｜authority｜>", "domain": "<｜domain｜>",
               "title": "<｜title｜>", "read_url": "<｜read_url｜>"}

EFFORT_PREAMBLE = {
    "low": "",
    "high": (
        "Reasoning Effort: Absolute maximum with no shortcuts permitted.\n"
        "You MUST be very thorough in your thinking and comprehensively decompose the problem to resolve the root cause, "
        "rigorously stress-testing your logic against all potential paths, edge cases, and adversarial scenarios.\n"
        "Explicitly write out your entire deliberation process, documenting every intermediate step, considered "
        "alternative, and rejected hypothesis to ensure absolutely no assumption is left unchecked.\n\n"),
    "max": (
        "Reasoning Effort: Beyond maximum — exhaustive, relentless, and uncompromising.\n"
        "You MUST reason with the utmost depth and rigor, leaving absolutely nothing to chance: exhaustively decompose the "
        "problem into its most fundamental components, trace every causal chain to its root, and resolve the underlying "
        "cause rather than any surface symptom.\n"
        "Do not stop reasoning until you have independently verified the solution from multiple angles and are certain "
        "that no assumption remains unchecked and no error remains undiscovered.\n\n"),
}
EFFORT_ALIAS = {None: "low", "minimal": "low", "medium": "low"}

_TOOLS_HEAD = (
    "## Tools\n\nYou have access to a set of tools to help answer the user's question. You can invoke tools by writing a "
    f"\"<{DSML}tool_calls>\" block like the following:\n\n"
    f"<{DSML}tool_calls>\n<{DSML}invoke name=\"$TOOL_NAME\">\n"
    f"<{DSML}parameter name=\"$PARAMETER_NAME\" string=\"true|false\">$PARAMETER_VALUE</{DSML}parameter>\n...\n"
    f"</{DSML}invoke>\n<{DSML}invoke name=\"$TOOL_NAME2\">\n...\n</{DSML}invoke>\n</{DSML}tool_calls>\n\n"
    "String parameters should be specified as is and set `string=\"true\"`. For all other types (numbers, booleans, "
    "arrays, objects), pass the value in JSON format and set `string=\"false\"`.\n\n"
    f"If thinking_mode is enabled (triggered by {THINK_OPEN}), you MUST output your complete reasoning inside "
    f"{THINK_OPEN}...{THINK_CLOSE} BEFORE any tool calls or final response.\n\n"
    f"Otherwise, output directly after {THINK_CLOSE} with tool calls or final response.\n\n"
    "### Available Tool Schemas\n\n")
_TOOLS_TAIL = "\n\nYou MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls.\n"


def _json(v: Any) -> str:
    try:
        return json.dumps(v, ensure_ascii=False)
    except UnicodeEncodeError:
        return json.dumps(v, ensure_ascii=True)


def _tool_catalogue(tools: list[dict]) -> str:
    return _TOOLS_HEAD + "\n".join(_json(t.get("function", t)) for t in tools) + _TOOLS_TAIL


def _dsml_calls(tool_calls: list[dict]) -> str:
    blocks = []
    for tc in tool_calls:
        fn = tc.get("function", tc)
        raw = fn.get("arguments", "{}")
        try:
            args = json.loads(raw) if isinstance(raw, str) else dict(raw)
        except Exception:
            args = {"arguments": raw}
        params = "\n".join(
            f"<{DSML}parameter name=\"{k}\" string=\"{'true' if isinstance(v, str) else 'false'}\">"
            f"{v if isinstance(v, str) else _json(v)}</{DSML}parameter>" for k, v in args.items())
        blocks.append(f"<{DSML}invoke name=\"{fn.get('name')}\">\n{params}\n</{DSML}invoke>")
    return f"\n\n<{DSML}tool_calls>\n" + "\n".join(blocks) + f"\n</{DSML}tool_calls>"


def _text(content: Any) -> str:
    if isinstance(content, list):
        return "\n\n".join(p.get("text", "") if p.get("type") == "text" else f"[Unsupported {p.get('type')}]"
                           for p in content if isinstance(p, dict))
    return content or ""


def _fold_tool_results(messages: list[dict]) -> list[dict]:
    """Tool-role messages -> ``tool_result`` parts of user turns, ordered like the calls of the preceding assistant."""
    out: list[dict] = []
    order: dict[str, int] = {}
    for m in messages:
        m = copy.deepcopy(m)
        role = m.get("role")
        if role == "assistant":
            order = {tc.get("id", ""): i for i, tc in enumerate(m.get("tool_calls") or [])}
            out.append(m)
        elif role == "tool":
            part = {"kind": "result", "id": m.get("tool_call_id", ""), "text": _text(m.get("content"))}
            if out and out[-1].get("role") == "user" and "parts" in out[-1]:
                out[-1]["parts"].append(part)
            else:
                out.append({"role": "user", "parts": [part]})
            out[-1]["_order"] = order
        elif role == "user":
            part = {"kind": "text", "text": _text(m.get("content"))}
            if out and out[-1].get("role") == "user" and "parts" in out[-1] and out[-1].get("task") is None and \
                    any(p["kind"] == "result" for p in out[-1]["parts"]):
                out[-1]["parts"].append(part)
            else:
                out.append({"role": "user", "parts": [part], **{k: m[k] for k in ("task", "wo_eos") if k in m}})
        else:
            out.append(m)
    for m in out:
        if m.get("role") == "user" and m.get("_order"):
            od = m.pop("_order")
            res = sorted((p for p in m["parts"] if p["kind"] == "result"), key=lambda p: od.get(p["id"], len(od)))
            it = iter(res)
            m["parts"] = [next(it) if p["kind"] == "result" else p for p in m["parts"]]
    return out


def render(messages: list[dict[str, Any]], tools: list[dict] | None = None, thinking: bool = False,
           reasoning_effort: str | None = None, add_generation_prompt: bool = True, add_bos: bool = True) -> str:
    """``messages`` in OpenAI form (roles system / developer / user / assistant / tool).  ``tools`` may also be given
    as a ``tools`` field of the system message, which is where the catalogue is printed."""
    msgs = _fold_tool_results(messages)
    if tools:
        if msgs and msgs[0].get("role") == "system":
            msgs[0] = dict(msgs[0], tools=tools)
        else:
            msgs.insert(0, {"role": "system", "content": "", "tools": tools})
    keep_all_reasoning = any(m.get("tools") for m in msgs)
    effort = EFFORT_ALIAS.get(reasoning_effort, reasoning_effort)
    if effort not in EFFORT_PREAMBLE:
        raise ValueError(f"invalid reasoning effort {reasoning_effort!r}")
    last_user = max((i for i, m in enumerate(msgs) if m.get("role") in ("user", "developer")), default=-1)
    out = BOS if add_bos else ""
    if thinking:
        out += EFFORT_PREAMBLE[effort]
    for i, m in enumerate(msgs):
        role = m.get("role")
        if role == "system":
            out += _text(m.get("content"))
            if m.get("tools"):
                out += "\n\n" + _tool_catalogue(m["tools"])
            if m.get("response_format"):
                out += "\n\n## Response Format:\n\nYou MUST strictly adhere to the following schema to reply:\n" + _json(m["response_format"])
        elif role == "developer":
            out += USER + _text(m.get("content"))
            if m.get("tools"):
                out += "\n\n" + _tool_catalogue(m["tools"])
        elif role == "user":
            out += USER + "\n\n".join(p["text"] if p["kind"] == "text" else f"<tool_result>{p['text']}</tool_result>"
                                      for p in m["parts"])
        elif role == "latest_reminder":
            out += LATEST_REMINDER + _text(m.get("content"))
        elif role == "assistant":
            after_task = i > 0 and msgs[i - 1].get("task") is not None     # a task answer carries no reasoning
            if thinking and not after_task and (keep_all_reasoning or i > last_user):
                out += (m.get("reasoning_content") or "") + THINK_CLOSE
            out += _text(m.get("content"))
            if m.get("tool_calls"):
                out += _dsml_calls(m["tool_calls"])
            if not m.get("wo_eos"):
                out += EOS
        else:
            raise ValueError(f"unknown role {role!r}")
        nxt = msgs[i + 1].get("role") if i + 1 < len(msgs) else None
        if (nxt is not None and nxt not in ("assistant", "latest_reminder")) or (nxt is None and not add_generation_prompt):
            continue
        task = m.get("task")
        if task is not None:
            if task not in TASK_TOKENS:
                raise ValueError(f"invalid task {task!r}")
            if task == "action":
                out += ASSISTANT + (THINK_OPEN if thinking else THINK_CLOSE)
            out += TASK_TOKENS[task]
        elif role in ("user", "developer"):
            out += ASSISTANT
            out += THINK_OPEN if thinking and (keep_all_reasoning or i >= last_user) else THINK_CLOSE
    return out


_INVOKE = re.compile(rf"<{DSML}invoke name=\"(?P<name>[^\"]*)\">(?P<body>.*?)</{DSML}invoke>", re.S)
_PARAM = re.compile(rf"<{DSML}parameter name=\"(?P<k>[^\"]*)\" string=\"(?P<s>true|false)\">(?P<v>.*?)</{DSML}parameter>", re.S)


def parse_completion(text: str, thinking: bool = False) -> dict[str, Any]:
    """Completion text (what follows the generation prompt) -> assistant message with ``reasoning_content``,
    ``content`` and OpenAI-style ``tool_calls`` (arguments as a JSON string)."""
    text = text.replace(EOS, "")
    reasoning = None
    if thinking or THINK_CLOSE in text:
        if THINK_CLOSE in text:
            reasoning, text = text.split(THINK_CLOSE, 1)
        else:
            reasoning, text = text, ""
        reasoning = reasoning.replace(THINK_OPEN, "")
    calls = []
    block = re.search(rf"<{DSML}tool_calls>(.*?)(</{DSML}tool_calls>|$)", text, re.S)
    if block:
        for n, m in enumerate(_INVOKE.finditer(block.group(1))):
            args: dict[str, Any] = {}
            for p in _PARAM.finditer(m.group("body")):
                v = p.group("v")
                if p.group("s") == "false":
                    try:
                        v = json.loads(v)
                    except Exception:
                        pass
                args[p.group("k")] = v
            calls.append({"id": f"call_{n}", "type": "function",
                          "function": {"name": m.group("name"), "arguments": _json(args)}})
        text = text[:block.start()]
    return {"role": "assistant", "content": text.strip("\n") if calls else text, "reasoning_content": reasoning,
            "tool_calls": calls or None}
