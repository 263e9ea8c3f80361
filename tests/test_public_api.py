"""Typed API, protocol normalisation and backend contract with a fake runtime (no GPU, no torch import)."""
import json
import sys

import pytest

import pocketllm
from pocketllm import (ConfigurationError, EngineArgs, GenerationRequest, SamplingParams, TimingMetrics,
                       UnsupportedFeatureError, Usage)
from pocketllm.backends.native_backend import NativeBackend
from pocketllm.protocol import chat as chatmod
from pocketllm.protocol.prompt import TokenizerHandle
from pocketllm.protocol.requests import build_chat_request, build_completion_request


class FakeRuntime:
    """Echo model: next token = (last token + 1) % 250; records every call in order."""
    eos_token_ids = (249,)
    max_context = 64
    supports_sampling = False

    def __init__(self):
        self.calls = []
        self.slots = set()
        self.last = {}

    def allocate(self):
        s = len(self.calls)
        self.slots.add(s)
        self.calls.append(("allocate", s))
        return s

    def free(self, slot):
        self.slots.discard(slot)
        self.calls.append(("free", slot))

    def prefill_tokens(self, slot, prompt, chunk, sp):
        self.calls.append(("prefill", slot, len(prompt), chunk))
        self.last[slot] = (prompt[-1] + 1) % 250
        return self.last[slot]

    def decode_tokens(self, slots, toks, sp):
        self.calls.append(("decode", tuple(slots), tuple(toks)))
        out = []
        for s, t in zip(slots, toks):
            self.last[s] = (t + 1) % 250
            out.append(self.last[s])
        return out


def make_backend(**kw):
    rt = FakeRuntime()
    return NativeBackend(EngineArgs(model="fake", **kw), runtime=rt), rt


def test_import_does_not_pull_torch():
    import subprocess
    code = "import sys, pocketllm; from pocketllm import EngineArgs, SamplingParams; assert 'torch' not in sys.modules"
    assert subprocess.run([sys.executable, "-c", code], cwd=".").returncode == 0


def test_engine_args_validation():
    with pytest.raises(ConfigurationError):
        EngineArgs(model="m", backend="nope")
    with pytest.raises(ConfigurationError):
        EngineArgs(model="m", tensor_parallel_size=2, tensor_parallel_rank=2)
    with pytest.raises(ConfigurationError):
        EngineArgs(model="m", kv_cache_dtype="fp3")
    assert EngineArgs(model="m", backend="CPP").backend == "cpp"


def test_engine_args_from_env(monkeypatch):
    monkeypatch.setenv("POCKETLLM_CHECKPOINT", "/ckpt")
    monkeypatch.setenv("POCKETLLM_TP_SIZE", "4")
    monkeypatch.setenv("TP_RANK", "3")
    monkeypatch.setenv("POCKETLLM_BACKEND_OPTIONS", json.dumps({"pd_mode": "serial"}))
    a = EngineArgs.from_env()
    assert (a.model, a.tensor_parallel_size, a.tensor_parallel_rank, a.backend_options) == ("/ckpt", 4, 3, {"pd_mode": "serial"})
    monkeypatch.setenv("POCKETLLM_TP_SIZE", "x")
    with pytest.raises(ConfigurationError):
        EngineArgs.from_env()


def test_sampling_params():
    sp = SamplingParams.from_openai({"max_completion_tokens": 7, "temperature": 0, "stop": "END"})
    assert sp.greedy and sp.max_tokens == 7 and sp.stop == ("END",)
    assert not SamplingParams(temperature=0.8).greedy
    for bad in ({"top_p": 0}, {"temperature": -1}, {"n": 17}, {"max_tokens": 0}, {"top_logprobs": 99}):
        with pytest.raises(ConfigurationError):
            SamplingParams.from_openai(bad)
    with pytest.raises(ConfigurationError):
        SamplingParams(stop=[str(i) for i in range(17)])


def test_timing_convention_first_token_counts_as_prefill():
    tm = TimingMetrics(prefill_seconds=2.0, decode_seconds=1.0)
    tp = tm.throughput(Usage(prompt_tokens=100, completion_tokens=11))
    assert tp["prefill_tps"] == 50.0 and tp["decode_tps"] == 10.0


def test_request_validation():
    with pytest.raises(ConfigurationError):
        GenerationRequest()
    with pytest.raises(ConfigurationError):
        GenerationRequest(prompt_tokens=[])
    with pytest.raises(ConfigurationError):
        GenerationRequest(prompt_tokens=[1, -2])
    assert GenerationRequest(prompt_tokens=(1, 2)).prompt_tokens == [1, 2]


def test_chat_normalisation():
    body = {"messages": [{"role": "developer", "content": [{"type": "text", "text": "be "}, {"type": "text", "text": "brief"}]},
                         {"role": "user", "content": "hi"}],
            "tools": [{"type": "function", "function": {"name": "get", "parameters": {"type": "object"}}}],
            "tool_choice": {"type": "function", "function": {"name": "get"}}, "reasoning_effort": "high", "stream": True}
    c = chatmod.ChatRequest.from_body(body)
    assert c.messages[0] == {"role": "system", "content": "be brief"}
    assert c.thinking and c.reasoning_effort == "high" and c.stream
    assert "get" in c.tool_instruction
    assert c.messages_with_instruction()[0]["content"].endswith("get.")
    with pytest.raises(ConfigurationError):
        chatmod.ChatRequest.from_body({"messages": [{"role": "robot", "content": "x"}]})
    with pytest.raises(ConfigurationError):
        chatmod.ChatRequest.from_body({"messages": [{"role": "user", "content": [{"type": "image_url"}]}]})
    with pytest.raises(ConfigurationError):
        chatmod.ChatRequest.from_body({"messages": [{"role": "user", "content": "x"}], "tools": [{"function": {"name": "a"}}],
                                       "tool_choice": {"function": {"name": "b"}}})


def test_stop_reasoning_and_tool_extraction():
    assert chatmod.truncate_at_stop("abcENDdef", ["zzz", "END"]) == ("abc", True)
    assert chatmod.held_back_suffix("hello EN", ["END"]) == 2
    assert chatmod.split_reasoning("<think>plan</think>answer") == ("plan", "answer")
    assert chatmod.split_reasoning("plan</think> answer") == ("plan", "answer")
    rest, calls = chatmod.extract_tool_calls('ok <tool_call>{"name": "get", "arguments": {"x": 1}}</tool_call>')
    assert rest == "ok" and calls[0]["function"]["name"] == "get" and json.loads(calls[0]["function"]["arguments"]) == {"x": 1}


def test_request_builders_with_byte_tokenizer():
    tok = TokenizerHandle(None, "bytes")
    req, chat = build_chat_request({"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3}, tok)
    assert tok.decode(req.prompt_tokens).endswith("<|assistant|>\n") and req.sampling_params.max_tokens == 3
    r2 = build_completion_request({"prompt": [1, 2, 3]}, tok)
    assert r2.prompt_tokens == [1, 2, 3]
    with pytest.raises(ConfigurationError):
        build_completion_request({"prompt": ""}, tok)


def test_backend_generate_order_and_eos():
    b, rt = make_backend()
    res = b.generate([GenerationRequest(prompt_tokens=[10, 245], sampling_params=SamplingParams(max_tokens=10))])[0]
    # 246 247 248 then 249 == eos -> stop, eos not returned
    assert res.token_ids == [246, 247, 248] and res.finish_reason == "stop"
    assert res.usage.prompt_tokens == 2 and res.usage.completion_tokens == 3
    kinds = [c[0] for c in rt.calls]
    assert kinds == ["allocate", "prefill", "decode", "decode", "decode", "free"]
    assert not rt.slots


def test_backend_length_stop_strings_and_context_clamp():
    b, rt = make_backend()
    r = b.generate([GenerationRequest(prompt_tokens=[64], sampling_params=SamplingParams(max_tokens=4))])[0]
    assert r.token_ids == [65, 66, 67, 68] and r.finish_reason == "length" and r.text == "ABCD"
    r = b.generate([GenerationRequest(prompt_tokens=[64], sampling_params=SamplingParams(max_tokens=20, stop=("CD",)))])[0]
    assert r.text == "AB" and r.finish_reason == "stop"
    long_prompt = list(range(60))
    r = b.generate([GenerationRequest(prompt_tokens=long_prompt, sampling_params=SamplingParams(max_tokens=50))])[0]
    assert len(r.token_ids) == 4           # clamped by max_context 64
    with pytest.raises(ConfigurationError):
        b.generate([GenerationRequest(prompt_tokens=list(range(64)))])


def test_backend_rejects_unsupported_features():
    b, _ = make_backend()
    with pytest.raises(UnsupportedFeatureError):
        b.generate([GenerationRequest(prompt_tokens=[1], sampling_params=SamplingParams(temperature=0.7))])
    with pytest.raises(UnsupportedFeatureError):
        b.generate([GenerationRequest(prompt_tokens=[1], sampling_params=SamplingParams(logprobs=True))])


def test_stream_events_and_llm_facade():
    b, _ = make_backend()
    llm = pocketllm.LLM(backend=b)
    evs = list(llm.generate_stream([72], SamplingParams(max_tokens=3)))
    assert "".join(e.text for e in evs) == "IJK"
    assert evs[-1].finish_reason == "length" and evs[-1].usage.completion_tokens == 3
    out = llm.generate(["A", "B"], SamplingParams(max_tokens=1))
    assert [o.text for o in out] == ["B", "C"]
    assert llm.health().ready
    llm.close()
    assert llm.health().status == "closed"


def test_tp_fanout_order_matches_local_calls():
    """Rank 0 must send each command to the workers before running it locally."""
    log = []

    class Chan:
        world = 2

        def send(self, op, *payload):
            log.append(("send", op))

    rt = FakeRuntime()
    orig_prefill, orig_decode = rt.prefill_tokens, rt.decode_tokens
    rt.prefill_tokens = lambda *a: (log.append(("local", 3)), orig_prefill(*a))[1]
    rt.decode_tokens = lambda *a: (log.append(("local", 4)), orig_decode(*a))[1]
    b = NativeBackend(EngineArgs(model="fake", tensor_parallel_size=2), runtime=rt, channel=Chan())
    b.generate([GenerationRequest(prompt_tokens=[5], sampling_params=SamplingParams(max_tokens=3))])
    ops = [x for x in log if x[1] in (3, 4)]
    assert ops == [("send", 3), ("local", 3), ("send", 4), ("local", 4), ("send", 4), ("local", 4)]


def test_worker_loop_mirrors_commands_and_survives_errors():
    from pocketllm.backends.native_backend import OP_ALLOC, OP_DECODE, OP_FREE, OP_PREFILL, OP_STOP

    class Chan:
        world = 2

        def __init__(self, msgs):
            self.msgs = list(msgs)

        def recv(self):
            return self.msgs.pop(0)

    rt = FakeRuntime()
    msgs = [(OP_ALLOC,), (OP_PREFILL, 0, 8192, [1, 2]), (OP_DECODE, 0, 3), (OP_DECODE, 99, "bad"), (OP_FREE, 0), (OP_STOP,)]
    b = NativeBackend(EngineArgs(model="fake", tensor_parallel_size=2, tensor_parallel_rank=1), runtime=rt, channel=Chan(msgs))
    b.run_worker()
    assert [c[0] for c in rt.calls] == ["allocate", "prefill", "decode", "decode", "free"] or \
        [c[0] for c in rt.calls] == ["allocate", "prefill", "decode", "free"]


def test_loader_refuses_an_unimplemented_speculative_method_before_touching_a_device():
    from deepseek_v4_2080ti_b200.runtime import loader
    from pocketllm.api.errors import ConfigurationError
    args = EngineArgs(model="synthetic:qwen-tiny", speculative_method="dspark")
    with pytest.raises(ConfigurationError, match="speculative_method"):
        loader.load_runtime(args)
    args = EngineArgs(model="/nonexistent/model.gguf", speculative_method="mtp")
    with pytest.raises(ConfigurationError, match="hybrid runtime"):
        loader.load_runtime(args)


class _FakeGgufRuntime:
    """next token = (last token + 1) % 50; records the largest decode batch."""

    def __init__(self, single):
        self.single_sequence = single
        self.free_ids, self.last, self.max_batch = [2, 1, 0], {}, 0

    def allocate(self):
        return self.free_ids.pop()

    def free(self, slot):
        self.free_ids.append(slot)
        self.last.pop(slot)

    def prefill(self, slot, ids, chunk):
        import torch
        self.last[slot] = int(ids[-1])
        return torch.tensor([(self.last[slot] + 1) % 50])

    def decode(self, slots, toks):
        import torch
        self.max_batch = max(self.max_batch, len(slots))
        return torch.tensor([(int(t) + 1) % 50 for t in toks.tolist()])


@pytest.mark.parametrize("single", [False, True])
def test_gguf_runtime_adapter_batches_up_to_the_runtime_slots(single):
    from deepseek_v4_2080ti_b200.runtime.loader import GgufRuntimeAdapter, _is_gguf
    rt = _FakeGgufRuntime(single)
    ad = GgufRuntimeAdapter(rt, 128, 3, "cpu")
    assert ad.max_slots == (1 if single else 3) and not ad.supports_sampling
    res = ad.generate_batch([[1, 2, 3], [10], [48], [7, 8]], [4, 2, 5, 3], {0}, 8)
    assert res[0][0] == [4, 5, 6, 7] and res[0][1] == "length"
    assert res[1][0] == [11, 12] and res[3][0] == [9, 10, 11]
    assert res[2][0] == [49] and res[2][1] == "stop"          # 48 -> 49 -> 0 (eos, dropped)
    assert rt.max_batch == (1 if single else 3) and sorted(rt.free_ids) == [0, 1, 2] and ad.stats()["slots_free"] == ad.max_slots
    s = ad.allocate()
    if single:
        with pytest.raises(RuntimeError):
            ad.allocate()
    ad.prefill_tokens(s, [5], 0, None)
    assert ad.decode_tokens([s], [6], None) == [7]
    ad.free(s)
    assert _is_gguf("model.gguf") and not _is_gguf("/nonexistent/dir")


def test_response_format_travels_as_an_instruction_in_chat_prompts_only():
    from pocketllm.protocol.chat import ChatRequest, response_format_schema
    from deepseek_v4_2080ti_b200 import encoding
    schema = {"type": "object", "properties": {"x": {"type": "number"}}, "required": ["x"]}
    assert response_format_schema(None) is None and response_format_schema({"type": "text"}) is None
    assert response_format_schema({"type": "json_object"}) == {"type": "object"}
    assert response_format_schema({"type": "json_schema", "json_schema": {"name": "p", "schema": schema}}) == schema
    with pytest.raises(ConfigurationError):
        response_format_schema({"type": "yaml"})
    body = {"messages": [{"role": "user", "content": "a point"}],
            "response_format": {"type": "json_schema", "json_schema": {"name": "p", "schema": schema}}}
    chat = ChatRequest.from_body(body)
    native = encoding.render_chat("deepseek_v4", chat.messages_with_instruction(True))
    assert "## Response Format:" in native and '"required": ["x"]' in native and native.index("Response Format") < native.index("a point")
    other = encoding.render_chat("glm_dsa", chat.messages_with_instruction(False))
    assert "strictly follows this JSON schema" in other and '"required": ["x"]' in other
    # an existing system message keeps its text; the tool instruction and the schema share it
    body["messages"].insert(0, {"role": "system", "content": "Be brief."})
    body["response_format"] = {"type": "json_object"}
    msgs = ChatRequest.from_body(body).messages_with_instruction(False)
    assert msgs[0]["content"].startswith("Be brief.") and "valid JSON object" in msgs[0]["content"] and len(msgs) == 2
    assert ChatRequest.from_body({"messages": body["messages"]}).messages_with_instruction() == ChatRequest.from_body({"messages": body["messages"]}).messages
    # through the builders: a chat request is accepted, a raw completion with a schema is refused
    tok = TokenizerHandle.load(None)
    req, _ = build_chat_request(body, tok)
    assert req.metadata["response_format_in_prompt"] and b"valid JSON object" in bytes(req.prompt_tokens)
    rt = FakeRuntime()
    rt.max_context = 512
    backend = NativeBackend(EngineArgs(model="fake"), runtime=rt)
    req.sampling_params.max_tokens = 2
    assert len(backend.generate([req])[0].token_ids) == 2
    raw = build_completion_request({"prompt": "A", "response_format": {"type": "json_object"}, "max_tokens": 2}, tok)
    with pytest.raises(UnsupportedFeatureError, match="chat request"):
        backend.generate([raw])


def test_n_choices_expand_with_consecutive_seeds_and_merge():
    from pocketllm.protocol.requests import expand_choices, merge_choices
    req = GenerationRequest(prompt_tokens=[5], sampling_params=SamplingParams(max_tokens=2, n=3, seed=10, temperature=0.0),
                            request_id="r")
    parts = expand_choices(req)
    assert [p.request_id for p in parts] == ["r-0", "r-1", "r-2"] and [p.sampling_params.seed for p in parts] == [10, 11, 12]
    assert all(p.sampling_params.n == 1 for p in parts) and req.sampling_params.n == 3
    assert expand_choices(GenerationRequest(prompt_tokens=[5]))[0].sampling_params.n == 1
    b, rt = make_backend()
    (res,) = b.generate([req])
    assert res.request_id == "r" and len(res.choices) == 3 and res.token_ids == res.choices[0].token_ids == [6, 7]
    assert res.usage.prompt_tokens == 1 and res.usage.completion_tokens == 6 and res.choices[1].choices == []
    assert sum(1 for c in rt.calls if c[0] == "prefill") == 3
    # mixed with an ordinary request: order and grouping are kept
    a, b2 = b.generate([GenerationRequest(prompt_tokens=[1], sampling_params=SamplingParams(max_tokens=1)), req])
    assert a.choices == [] and a.token_ids == [2] and len(b2.choices) == 3
    with pytest.raises(ConfigurationError):
        SamplingParams(n=0)
    with pytest.raises(UnsupportedFeatureError):
        list(b.stream(req))


def test_token_ids_outside_the_vocabulary_never_reach_the_runtime():
    b, rt = make_backend()
    rt.vocab_size = 250
    for bad in ([1, -1], [250], [2 ** 31]):                        # refused by the request type or by the backend
        with pytest.raises(ConfigurationError):
            b.generate([GenerationRequest(prompt_tokens=bad, sampling_params=SamplingParams(max_tokens=1))])
    with pytest.raises(ConfigurationError, match="not a token id of this model"):
        b.generate([GenerationRequest(prompt_tokens=[3, 250], sampling_params=SamplingParams(max_tokens=1))])
    assert not any(c[0] == "prefill" for c in rt.calls)
    assert b.generate([GenerationRequest(prompt_tokens=[0, 249], sampling_params=SamplingParams(max_tokens=1))])[0].token_ids == [0]
    del rt.vocab_size                                    # a runtime that does not say: still whole and non-negative
    with pytest.raises(ConfigurationError):
        b.generate([GenerationRequest(prompt_tokens=[-5], sampling_params=SamplingParams(max_tokens=1))])
