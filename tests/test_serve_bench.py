"""The load generator against a live server on the host path: every request answered, figures consistent."""
import json
import threading

from pocketllm import LLM, EngineArgs
from pocketllm.server.openai import make_server
from deepseek_v4_2080ti_b200.utils import serve_bench as sb


def test_levels_against_the_host_server(capsys):
    llm = LLM(EngineArgs(model="synthetic:qwen-tiny", device="cpu", max_model_len=128))
    httpd, _ = make_server(llm.backend, "127.0.0.1", 0, "tiny")
    threading.Thread(target=httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True).start()
    port = httpd.server_address[1]
    try:
        row = sb.run_level("127.0.0.1", port, 2, 4, prompt_tokens=8, max_tokens=5, vocab=500, seed=1)
        assert row["ok"] == 4 and row["errors"] == 0 and row["generated_tokens_per_second"] > 0
        assert 0 < row["ttft_median_s"] <= row["latency_median_s"] <= row["latency_p90_s"] <= row["wall_seconds"]
        plain = sb.run_level("127.0.0.1", port, 1, 2, prompt_tokens=8, max_tokens=3, vocab=500, seed=1, stream=False)
        assert plain["ok"] == 2 and plain["generated_tokens_per_second"] > 0
        # a prompt that does not fit is an error row, not an exception
        bad = sb.run_level("127.0.0.1", port, 1, 1, prompt_tokens=400, max_tokens=3, vocab=500, seed=1)
        assert bad["ok"] == 0 and bad["errors"] == 1 and "HTTP 400" in bad["first_error"]
        assert sb.main(["--url", f"http://127.0.0.1:{port}", "--concurrency", "1,2", "--requests", "2", "--prompt-tokens", "6",
                        "--max-tokens", "3", "--vocab", "500"]) == 0
        lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
        assert [l["concurrency"] for l in lines] == [1, 2] and lines[0]["speedup_vs_first_level"] == 1.0
    finally:
        httpd.shutdown()
        httpd.server_close()
        llm.close()
    assert sb.run_level("127.0.0.1", port, 1, 1, 4, 2, 100, 0, timeout=2)["errors"] == 1      # nobody listens any more


def test_against_the_native_server_with_token_id_answers():
    import pytest
    cpp = pytest.importorskip("deepseek_v4_2080ti_b200.pocketllm_cpp")
    from tests.test_native_http_server import FakeEngine
    eng = FakeEngine()
    opt = cpp.OpenAIServerOptions()
    opt.port = 0
    srv = cpp.OpenAIServer(eng, opt)
    srv.start()
    try:
        for stream, route in ((False, "/v1/completions"), (True, "/v1/chat/completions")):
            row = sb.run_level("127.0.0.1", srv.port, 3, 6, prompt_tokens=5, max_tokens=4, vocab=40, seed=2, stream=stream, route=route)
            assert row["ok"] == 6 and row["errors"] == 0 and row["generated_tokens_per_second"] > 0, row
    finally:
        srv.stop()
