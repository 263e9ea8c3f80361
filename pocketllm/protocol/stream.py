"""Incremental splitter for streamed chat completions: routes text deltas into ``reasoning_content`` and ``content``
and keeps tool-call markup out of the visible stream.

It is a small state machine over the text that has arrived so far:

* REASONING: everything up to ``</think>`` is reasoning.  The stream starts here when the request enabled thinking
  (the template has already opened the block) or when the completion itself opens with ``<think>``.
* CONTENT: visible answer text.  The first tool-call opener (``<tool_call>`` or the DSML ``<｜DSML｜tool_calls`` block
  with its two leading newlines) ends it.
* TOOLS: nothing more is shown; the tail is kept and parsed at the end into OpenAI ``tool_calls``.

A chunk boundary can fall inside a marker, so text that could still turn out to be the beginning of a marker is held
back until the next delta decides it.  Behaviour covered: the reference's streaming decoder
(src/server/openai.py:514-585: reasoning before ``</think>``, content after it, truncation at the tool-call block,
held-back partial markers), restated over deltas instead of re-decoding the whole token list on every step.
"""
from __future__ import annotations

from typing import Any

from .chat import extract_tool_calls

DSML = "｜DSML｜"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
TOOL_OPENERS = ("<tool_call>", f"\n\n<{DSML}tool_calls", f"<{DSML}tool_calls")


def _held(text: str, markers: tuple[str, ...]) -> int:
    """Length of the longest suffix of ``text`` that is a proper prefix of one of ``markers``."""
    best = 0
    for m in markers:
        for n in range(min(len(text), len(m) - 1), best, -1):
            if text.endswith(m[:n]):
                best = n
                break
    return best


def _dsml_tool_calls(block: str) -> list[dict[str, Any]]:
    import json
    import re
    import uuid
    calls = []
    for inv in re.finditer(rf"<{DSML}invoke name=\"([^\"]+)\">(.*?)</{DSML}invoke>", block, re.S):
        args: dict[str, Any] = {}
        for par in re.finditer(rf"<{DSML}parameter name=\"([^\"]+)\" string=\"(true|false)\">(.*?)</{DSML}parameter>",
                               inv.group(2), re.S):
            raw = par.group(3)
            if par.group(2) == "true":
                args[par.group(1)] = raw
            else:
                try:
                    args[par.group(1)] = json.loads(raw)
                except json.JSONDecodeError:
                    args[par.group(1)] = raw
        calls.append({"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function",
                      "function": {"name": inv.group(1), "arguments": json.dumps(args, ensure_ascii=False)}})
    return calls


class StreamSplitter:
    """``feed(delta)`` returns the OpenAI delta objects to emit now; ``finish()`` flushes what was held back and
    returns ``(deltas, tool_calls)``."""

    def __init__(self, thinking: bool = False, tools: bool = False):
        self.state = "reasoning" if thinking else "start"
        self.tools = tools
        self.buf = ""               # text not yet classified or emitted
        self.reasoning = ""
        self.content = ""
        self.tool_text = ""

    # -- helpers
    def _emit(self, out: list[dict[str, str]], key: str, text: str) -> None:
        if not text:
            return
        if key == "content":
            self.content += text
        else:
            self.reasoning += text
        if out and key in out[-1] and len(out[-1]) == 1:
            out[-1][key] += text
        else:
            out.append({key: text})

    def feed(self, delta: str) -> list[dict[str, str]]:
        out: list[dict[str, str]] = []
        self.buf += delta
        while True:
            if self.state == "start":
                lead = self.buf.lstrip()
                if lead.startswith(THINK_OPEN):
                    self.buf = lead[len(THINK_OPEN):]
                    self.state = "reasoning"
                elif THINK_OPEN.startswith(lead):       # empty so far, or could still become "<think>"
                    return out
                else:
                    self.state = "content"
                continue
            if self.state == "reasoning":
                i = self.buf.find(THINK_CLOSE)
                if i >= 0:
                    self._emit(out, "reasoning_content", self.buf[:i])
                    self.buf = self.buf[i + len(THINK_CLOSE):]
                    self.state = "content"
                    continue
                keep = _held(self.buf, (THINK_CLOSE,))
                self._emit(out, "reasoning_content", self.buf[:len(self.buf) - keep])
                self.buf = self.buf[len(self.buf) - keep:]
                return out
            if self.state == "content":
                if not self.content:
                    self.buf = self.buf.lstrip("\n") if self.reasoning else self.buf
                hits = [(self.buf.find(m), m) for m in TOOL_OPENERS if self.tools and m in self.buf]
                if hits:
                    i, _ = min(hits)
                    self._emit(out, "content", self.buf[:i])
                    self.tool_text = self.buf[i:]
                    self.buf = ""
                    self.state = "tools"
                    return out
                keep = _held(self.buf, TOOL_OPENERS) if self.tools else 0
                self._emit(out, "content", self.buf[:len(self.buf) - keep])
                self.buf = self.buf[len(self.buf) - keep:]
                return out
            # tools: swallow
            self.tool_text += self.buf
            self.buf = ""
            return out

    def finish(self) -> tuple[list[dict[str, str]], list[dict[str, Any]]]:
        out: list[dict[str, str]] = []
        if self.state == "start":
            self.state = "content"
        if self.state == "reasoning":
            self._emit(out, "reasoning_content", self.buf)
        elif self.state == "content":
            self._emit(out, "content", self.buf)        # a held-back prefix that never completed is ordinary text
        else:
            self.tool_text += self.buf
        self.buf = ""
        calls: list[dict[str, Any]] = []
        if self.tool_text:
            if DSML in self.tool_text:
                calls = _dsml_tool_calls(self.tool_text)
            else:
                _, calls = extract_tool_calls(self.tool_text)
            if not calls:                               # markup that does not parse is shown rather than lost
                self._emit(out, "content", self.tool_text)
        return out, calls
