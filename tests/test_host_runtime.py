"""The host path of the public API (device="cpu"): the fp32 oracle of the Qwen-style hybrid behind the serving backend,
with every drafter of the speculative loop; the tokens are the oracle's greedy tokens whichever drafter proposes."""
import json

import pytest
import torch

from pocketllm import LLM, ConfigurationError, EngineArgs, SamplingParams, UnsupportedFeatureError
from deepseek_v4_2080ti_b200.formats import safetensors_io
from deepseek_v4_2080ti_b200.models import qwen_dspark_ref as ds
from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef

PROMPT = [3, 17, 99, 4, 250, 31, 8, 77, 12, 5]


def _greedy(n):
    cfg = qh.QwenHybridConfig.tiny()
    ref = QwenHybridRef(cfg, dict(qh.synth_state(cfg, 0, "cpu", std=0.05)))
    ids, out = list(PROMPT), []
    for _ in range(n):
        out.append(int(ref.forward(torch.tensor(ids))[-1].argmax()))
        ids.append(out[-1])
    return out


@pytest.fixture(scope="module")
def greedy():
    return _greedy(9)


@pytest.mark.parametrize("method", [None, "ngram", "mtp", "dspark", "dflash2"])
def test_every_drafter_serves_the_greedy_tokens(method, greedy):
    llm = LLM(EngineArgs(model="synthetic:qwen-tiny", device="cpu", max_model_len=128, speculative_method=method,
                         speculative_tokens=3))
    (res,) = llm.generate([PROMPT], SamplingParams(max_tokens=9, logprobs=True, top_logprobs=2))
    assert res.token_ids == greedy and res.usage.completion_tokens == 9
    assert len(res.logprobs) == 9 and all(e["logprob"] <= 0 and len(e["top_logprobs"]) == 2 for e in res.logprobs)
    assert all(e["top_logprobs"][0]["token_id"] == t for e, t in zip(res.logprobs, res.token_ids))     # greedy: the best token
    st = llm.backend.runtime.stats()
    if method in ("mtp", "dspark", "dflash2"):
        assert st["spec_rounds"] > 0 and st["spec_drafted"] >= st["spec_accepted"]
    if method is None:
        assert st["target_passes"] == 9 and st["spec_rounds"] == 0         # the last token needs no further pass
    # a second request reuses the slot
    (again,) = llm.generate([PROMPT], SamplingParams(max_tokens=4))
    assert again.token_ids == greedy[:4]
    llm.close()


def test_drafter_checkpoint_from_a_directory_and_refusals(tmp_path, greedy):
    cfg = qh.QwenHybridConfig.tiny()
    dcfg = ds.QwenDSparkConfig(hidden_size=cfg.hidden_size, intermediate_size=64, vocab_size=cfg.vocab_size, num_hidden_layers=1,
                               num_attention_heads=2, num_key_value_heads=1, head_dim=32, block_size=4,
                               mask_token_id=0, markov_rank=8, target_layer_ids=[1], original_max_position_embeddings=64)
    (tmp_path / "config.json").write_text(json.dumps(dcfg.to_json()))
    safetensors_io.write_file(str(tmp_path / "model.safetensors"), ds.synth_dspark_weights(dcfg, 3))
    llm = LLM(EngineArgs(model="synthetic:qwen-tiny", device="cpu", max_model_len=128, speculative_method="dspark",
                         speculative_tokens=8, backend_options={"drafter": str(tmp_path)}))
    (res,) = llm.generate([PROMPT], SamplingParams(max_tokens=9))
    assert res.token_ids == greedy
    assert llm.backend.runtime.block == 4                                  # clamped to the drafter's block
    llm.close()
    bad = dcfg.to_json(); bad["hidden_size"] = 2 * cfg.hidden_size
    (tmp_path / "config.json").write_text(json.dumps(bad))
    with pytest.raises((ConfigurationError, ValueError)):
        LLM(EngineArgs(model="synthetic:qwen-tiny", device="cpu", speculative_method="dspark",
                       backend_options={"drafter": str(tmp_path)})).generate([PROMPT], SamplingParams(max_tokens=1))
    with pytest.raises(UnsupportedFeatureError, match="greedy"):
        LLM(EngineArgs(model="synthetic:qwen-tiny", device="cpu")).generate([PROMPT], SamplingParams(max_tokens=2, temperature=0.8))


@pytest.mark.parametrize("method", ["mtp", "dspark"])
def test_the_adaptive_gate_changes_the_passes_not_the_tokens(method, greedy):
    llm = LLM(EngineArgs(model="synthetic:qwen-tiny", device="cpu", max_model_len=128, speculative_method=method,
                         speculative_tokens=3, backend_options={"spec_gate": "1"}))
    (res,) = llm.generate([PROMPT], SamplingParams(max_tokens=9))
    assert res.token_ids == greedy
    st = llm.backend.runtime.stats()
    assert any(k.startswith("spec_gate_") for k in st) and st["spec_gate_rounds"] + st.get("spec_gate_skipped", 0) >= 1
    llm.close()


def test_a_stream_delivers_log_probabilities_with_its_closing_chunk():
    import http.client
    import threading
    from pocketllm.server.openai import make_server
    llm = LLM(EngineArgs(model="synthetic:qwen-tiny", device="cpu", max_model_len=128))
    httpd, _ = make_server(llm.backend, "127.0.0.1", 0, "tiny")
    threading.Thread(target=httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True).start()
    try:
        c = http.client.HTTPConnection("127.0.0.1", httpd.server_address[1], timeout=60)
        c.request("POST", "/v1/completions", body=json.dumps({"prompt": PROMPT, "max_tokens": 4, "stream": True, "logprobs": 2}),
                  headers={"Content-Type": "application/json"})
        raw = c.getresponse().read().decode()
        c.close()
        chunks = [json.loads(l[6:]) for l in raw.splitlines() if l.startswith("data: ") and l != "data: [DONE]"]
        last = chunks[-1]["choices"][0]
        assert last["finish_reason"] == "length" and len(last["logprobs"]["token_logprobs"]) == 4
        assert all(lp <= 0 for lp in last["logprobs"]["token_logprobs"]) and len(last["logprobs"]["top_logprobs"][0]) == 2
        assert all("logprobs" not in ch["choices"][0] or ch is chunks[-1] for ch in chunks)
    finally:
        httpd.shutdown()
        httpd.server_close()
        llm.close()
