"""Log-probabilities of generated tokens: API result, OpenAI payloads (chat and legacy completions), refusal where the
runtime cannot report them; and on the GPU against the soft-max of the runtime's own logits."""
import http.client
import json
import math
import threading

import pytest

from pocketllm import LLM, EngineArgs, SamplingParams
from pocketllm.api.errors import UnsupportedFeatureError
from pocketllm.backends.native_backend import NativeBackend
from tests.test_public_api import FakeRuntime


class FakeWithLogprobs(FakeRuntime):
    supports_logprobs = True

    def token_logprobs(self, slot, token, top_n):
        # the chosen token has probability 1/2, the next ids share the rest
        top = [(token, math.log(0.5))] + [((token + j) % 250, math.log(0.5 / 2 ** j)) for j in range(1, top_n)]
        return {"logprob": math.log(0.5), "top": top[:top_n]}


def test_api_result_carries_one_entry_per_token():
    llm = LLM(backend=NativeBackend(EngineArgs(model="fake"), runtime=FakeWithLogprobs()))
    res = llm.generate([{"prompt_token_ids": [5, 6, 7]}], SamplingParams(max_tokens=4, logprobs=True, top_logprobs=3))[0]
    assert list(res.token_ids) == [8, 9, 10, 11] and len(res.logprobs) == 4
    e = res.logprobs[1]
    assert e["token_id"] == 9 and abs(e["logprob"] - math.log(0.5)) < 1e-12 and isinstance(e["token"], str)
    assert [a["token_id"] for a in e["top_logprobs"]] == [9, 10, 11] and abs(e["top_logprobs"][2]["logprob"] - math.log(0.125)) < 1e-12
    plain = llm.generate([{"prompt_token_ids": [5, 6, 7]}], SamplingParams(max_tokens=2))[0]
    assert plain.logprobs is None


def test_runtime_without_logprobs_refuses():
    llm = LLM(backend=NativeBackend(EngineArgs(model="fake"), runtime=FakeRuntime()))
    with pytest.raises(UnsupportedFeatureError):
        llm.generate([{"prompt_token_ids": [1]}], SamplingParams(max_tokens=2, logprobs=True))


def test_openai_payloads():
    from pocketllm.server.openai import make_server
    backend = NativeBackend(EngineArgs(model="fake"), runtime=FakeWithLogprobs())
    httpd, _ = make_server(backend, "127.0.0.1", 0, "fake-model")
    threading.Thread(target=httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True).start()
    try:
        def post(path, body):
            c = http.client.HTTPConnection("127.0.0.1", httpd.server_address[1], timeout=10)
            c.request("POST", path, body=json.dumps(body), headers={"Content-Type": "application/json"})
            r = c.getresponse()
            out = json.loads(r.read())
            c.close()
            return r.status, out
        st, out = post("/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 3,
                                                "logprobs": True, "top_logprobs": 2})
        assert st == 200
        content = out["choices"][0]["logprobs"]["content"]
        assert len(content) == 3 and len(content[0]["top_logprobs"]) == 2 and content[0]["bytes"] == list(content[0]["token"].encode())
        assert abs(content[0]["logprob"] - math.log(0.5)) < 1e-9
        st, out = post("/v1/completions", {"prompt": "abc", "max_tokens": 3, "logprobs": True, "top_logprobs": 2})
        lp = out["choices"][0]["logprobs"]
        assert st == 200 and len(lp["tokens"]) == len(lp["token_logprobs"]) == len(lp["top_logprobs"]) == len(lp["text_offset"]) == 3
        assert lp["text_offset"][0] == 0 and all(isinstance(d, dict) and len(d) <= 2 for d in lp["top_logprobs"])
        st, out = post("/v1/completions", {"prompt": "abc", "max_tokens": 2})
        assert st == 200 and out["choices"][0]["logprobs"] is None
    finally:
        httpd.shutdown()
        httpd.server_close()


@pytest.mark.gpu
def test_qwen_runtime_logprobs_are_the_softmax_of_its_logits():
    import torch
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.runtime.loader import RuntimeAdapter
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    w = qh.QwenHybridWeights(cfg, qh.synth_state(cfg, 0, "cuda", std=0.05), "cuda")
    rt = qh.QwenHybridRuntime(cfg, w, max_slots=1, max_context=256)
    llm = LLM(backend=NativeBackend(EngineArgs(model="synthetic:tiny", max_model_len=256), runtime=RuntimeAdapter(rt, 256)))
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(3)).tolist()
    res = llm.generate([{"prompt_token_ids": prompt}], SamplingParams(max_tokens=5, temperature=0.0, logprobs=True, top_logprobs=4))[0]
    assert len(res.logprobs) == 5
    for tok, e in zip(res.token_ids, res.logprobs):
        top = e["top_logprobs"]
        assert e["token_id"] == tok == top[0]["token_id"]                       # greedy: the chosen token leads the list
        assert abs(e["logprob"] - top[0]["logprob"]) < 1e-6 and e["logprob"] <= 0.0
        assert all(top[i]["logprob"] >= top[i + 1]["logprob"] for i in range(3))
        assert sum(math.exp(a["logprob"]) for a in top) <= 1.0 + 1e-5
    # the same request without logprobs yields the same tokens
    again = llm.generate([{"prompt_token_ids": prompt}], SamplingParams(max_tokens=5, temperature=0.0))[0]
    assert list(again.token_ids) == list(res.token_ids)
