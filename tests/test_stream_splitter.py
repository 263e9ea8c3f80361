"""Streaming chat splitter (pocketllm/protocol/stream.py) and its use by the SSE route: reasoning before </think>,
content after, tool-call markup withheld and delivered as tool_calls.  Behaviour of the reference's streaming
decoder (src/server/openai.py:514-585)."""
import http.client
import json
import threading

import pytest

from pocketllm.api.types import TokenEvent, Usage
from pocketllm.protocol.stream import DSML, StreamSplitter


def _run(text, cuts, **kw):
    sp = StreamSplitter(**kw)
    deltas = []
    prev = 0
    for c in list(cuts) + [len(text)]:
        deltas += sp.feed(text[prev:c])
        prev = c
    tail, calls = sp.finish()
    deltas += tail
    reasoning = "".join(d.get("reasoning_content", "") for d in deltas)
    content = "".join(d.get("content", "") for d in deltas)
    return reasoning, content, calls, deltas


def _all_single_cuts(text):
    return [[i] for i in range(1, len(text))]


def test_reasoning_then_content_for_every_cut_position():
    text = "step one\nstep two</think>\n\nThe answer is 4."
    for cuts in _all_single_cuts(text) + [list(range(1, len(text)))]:
        r, c, calls, deltas = _run(text, cuts, thinking=True)
        assert (r, c, calls) == ("step one\nstep two", "The answer is 4.", []), cuts
        assert all(len(d) == 1 for d in deltas)
        # no marker fragment ever leaks into either channel
        assert "<" not in r + c and "think" not in c


def test_completion_that_opens_its_own_think_block():
    text = "<think>hm</think>ok"
    for cuts in _all_single_cuts(text):
        assert _run(text, cuts)[:2] == ("hm", "ok"), cuts
    assert _run("plain <b>text</b>", [3])[:2] == ("", "plain <b>text</b>")
    assert _run("<thin air", [2])[:2] == ("", "<thin air")              # looked like a tag, was not
    assert _run("never closes", [4], thinking=True)[:2] == ("never closes", "")


def test_tool_call_json_block_is_withheld_and_parsed():
    text = 'Let me check.<tool_call>{"name": "get_weather", "arguments": {"city": "Paris"}}</tool_call>'
    for cuts in _all_single_cuts(text):
        r, c, calls, _ = _run(text, cuts, tools=True)
        assert c == "Let me check." and r == "", cuts
        assert len(calls) == 1 and calls[0]["function"]["name"] == "get_weather"
        assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}
    # without tools in the request the markup is ordinary text
    assert _run(text, [5], tools=False)[1] == text
    # an opener that never becomes a valid call is shown, not lost
    assert _run("a <tool_call>{broken", [3], tools=True)[1] == "a <tool_call>{broken"
    # a partial opener at the very end is ordinary text
    assert _run("a <tool", [2], tools=True)[1] == "a <tool"


def test_dsml_block_after_reasoning():
    block = (f'\n\n<{DSML}tool_calls>\n<{DSML}invoke name="search">\n<{DSML}parameter name="q" string="true">b200</{DSML}parameter>\n'
             f'<{DSML}parameter name="k" string="false">3</{DSML}parameter>\n</{DSML}invoke>\n</{DSML}tool_calls>')
    text = "think</think>Looking it up." + block
    for cuts in _all_single_cuts(text)[::3]:
        r, c, calls, _ = _run(text, cuts, thinking=True, tools=True)
        assert (r, c) == ("think", "Looking it up."), cuts
        assert [x["function"]["name"] for x in calls] == ["search"]
        assert json.loads(calls[0]["function"]["arguments"]) == {"q": "b200", "k": 3}


class _Tok:
    eos_token_id = 0
    has_chat_template = False

    def encode(self, text):
        return [1 + (ord(ch) % 200) for ch in text] or [1]

    def decode(self, ids):
        return "".join(chr(i) for i in ids)

    def apply_chat_template(self, messages, **kw):
        return "".join(str(m.get("content", "")) for m in messages)


class _ScriptedBackend:
    """Streams a fixed completion three characters at a time."""
    family = None

    def __init__(self, text):
        self.text, self.tokenizer, self.cancelled = text, _Tok(), []

    def prepare(self):
        pass

    def health(self):
        return {"status": "ok"}

    def stream(self, req):
        t = self.text
        for i in range(0, len(t), 3):
            last = i + 3 >= len(t)
            yield TokenEvent(req.request_id, text=t[i:i + 3], finish_reason="stop" if last else None,
                             usage=Usage(5, len(t)) if last else None)

    def cancel(self, rid):
        self.cancelled.append(rid)
        return False


def _sse(port, body):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request("POST", "/v1/chat/completions", body=json.dumps(body), headers={"Content-Type": "application/json"})
    r = c.getresponse()
    raw = r.read().decode()
    c.close()
    assert r.status == 200, raw
    events = [l[6:] for l in raw.split("\n\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    return [json.loads(e) for e in events[:-1]]


@pytest.fixture()
def scripted():
    from pocketllm.server.openai import make_server
    made = []

    def start(text):
        httpd, _ = make_server(_ScriptedBackend(text), "127.0.0.1", 0, "scripted")
        threading.Thread(target=httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True).start()
        made.append(httpd)
        return httpd.server_address[1]

    yield start
    for h in made:
        h.shutdown()
        h.server_close()


def test_sse_route_splits_reasoning_content_and_tool_calls(scripted):
    text = 'first I think</think>Calling.<tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>'
    port = scripted(text)
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}]
    chunks = _sse(port, {"messages": [{"role": "user", "content": "hi"}], "stream": True, "thinking": True, "tools": tools})
    deltas = [c["choices"][0]["delta"] for c in chunks]
    assert deltas[0] == {"role": "assistant", "content": ""}
    assert "".join(d.get("reasoning_content", "") for d in deltas) == "first I think"
    assert "".join(d.get("content", "") for d in deltas) == "Calling."
    calls = [d["tool_calls"] for d in deltas if "tool_calls" in d]
    assert len(calls) == 1 and calls[0][0]["index"] == 0 and calls[0][0]["function"]["name"] == "f"
    assert chunks[-1]["choices"][0]["finish_reason"] == "tool_calls" and chunks[-1]["usage"]["prompt_tokens"] == 5
    # the same completion without thinking or tools streams through untouched
    chunks = _sse(scripted("just text"), {"messages": [{"role": "user", "content": "hi"}], "stream": True})
    assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks) == "just text"
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop"


def test_any_chunking_gives_the_same_reasoning_content_and_tool_calls():
    """Property: how the text is cut into deltas never changes what comes out in total."""
    import random
    from pocketllm.protocol.stream import StreamSplitter
    texts = [
        ("<think>step one\nstep two</think>\n\nThe answer is 4.", True, False),
        ("plain answer with a < sign and </thin almost-marker", False, False),
        ("<think>plan</think>ok<tool_call>{\"name\": \"f\", \"arguments\": {\"x\": 1}}</tool_call>", False, True),
        ("reasoning continues</think>visible\n\n<｜DSML｜tool_calls>\n<｜DSML｜invoke name=\"g\">\n<｜DSML｜parameter name=\"q\" string=\"true\">hi</｜DSML｜parameter>\n</｜DSML｜invoke>\n</｜DSML｜tool_calls>", True, True),
        ("text <tool_cal not a call> more text", False, True),
    ]
    rng = random.Random(9)

    def run(text, thinking, tools, cuts):
        sp = StreamSplitter(thinking=thinking, tools=tools)
        deltas, last = [], 0
        for c in cuts + [len(text)]:
            deltas += sp.feed(text[last:c])
            last = c
        tail, calls = sp.finish()
        deltas += tail
        reasoning = "".join(d.get("reasoning_content", "") for d in deltas)
        content = "".join(d.get("content", "") for d in deltas)
        return reasoning, content, [(c["function"]["name"], c["function"]["arguments"]) for c in calls]
    for text, thinking, tools in texts:
        whole = run(text, thinking, tools, [])
        for _ in range(60):
            k = rng.randrange(1, min(12, len(text)))
            cuts = sorted(rng.sample(range(1, len(text)), k))
            assert run(text, thinking, tools, cuts) == whole, (text, cuts)
        assert run(text, thinking, tools, list(range(1, len(text)))) == whole          # one character at a time
