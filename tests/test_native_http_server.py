"""C++ OpenAI-compatible server and its Python sidecar client, on CPU: a Python fake engine behind the C++ batch
scheduler, real HTTP over a loopback socket, the JSON-lines helper as a real child process."""
import json
import os
import sys
import tempfile
import urllib.error
import urllib.request

import pytest

cpp = pytest.importorskip("deepseek_v4_2080ti_b200.pocketllm_cpp")


class FakeEngine(cpp.InferenceEngine):
    """next token = (sum of the slot's tokens + length) % 50; 49 is end-of-sequence."""

    def __init__(self, slots=4):
        super().__init__()
        self.sum, self.len, self.used = [0] * slots, [0] * slots, [False] * slots

    def max_slots(self): return len(self.used)
    def block_tokens(self): return 16
    def total_blocks(self): return 64
    def max_context(self): return 512
    def is_eos(self, t): return t == 49
    def reserve(self, slot, tokens): return tokens <= 512

    def allocate_slot(self):
        for i, u in enumerate(self.used):
            if not u:
                self.used[i], self.sum[i], self.len[i] = True, 0, 0
                return i
        return -1

    def free_slot(self, s): self.used[s] = False

    def batch_prefill(self, items):
        r = cpp.StepResult()
        out = []
        for it in items:
            self.sum[it.slot] += sum(it.tokens)
            self.len[it.slot] += len(it.tokens)
            out.append((self.sum[it.slot] + self.len[it.slot]) % 50 if it.last_chunk else -1)
        r.next_tokens = out
        return r

    def batch_decode(self, slots, tokens):
        r = cpp.StepResult()
        out = []
        for s, t in zip(slots, tokens):
            self.sum[s] += t
            self.len[s] += 1
            out.append((self.sum[s] + self.len[s]) % 50)
        r.next_tokens = out
        return r


def _expected(prompt, n):
    s, l, out = sum(prompt), len(prompt), []
    while len(out) < n:
        t = (s + l) % 50
        out.append(t)
        if t == 49:
            break
        s, l = s + t, l + 1
    return out


def _post(port, path, body):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=30) as r:
        return r.status, r.read().decode()


def test_http_routes_token_requests_and_errors():
    eng = FakeEngine()
    opt = cpp.OpenAIServerOptions()
    opt.port, opt.model_name = 0, "fake-model"
    srv = cpp.OpenAIServer(eng, opt)
    srv.start()
    try:
        port = srv.port
        assert port > 0
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=10) as r:
            h = json.loads(r.read())
        assert h["status"] == "ok" and h["sidecar"] == "none"
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/models", timeout=10) as r:
            assert json.loads(r.read())["data"][0]["id"] == "fake-model"
        prompt = [3, 7, 11]
        st, body = _post(port, "/v1/completions", {"prompt_token_ids": prompt, "max_tokens": 6})
        out = json.loads(body)
        want = _expected(prompt, 6)
        eos = want[-1] == 49
        assert st == 200 and out["choices"][0]["token_ids"] == (want[:-1] if eos else want)
        assert out["usage"]["prompt_tokens"] == 3 and out["object"] == "text_completion"
        st, body = _post(port, "/v1/chat/completions", {"prompt_token_ids": [1, 2], "max_tokens": 3, "stream": True})
        assert st == 200 and body.strip().endswith("data: [DONE]") and "chat.completion.chunk" in body
        for bad, code in (({"messages": [{"role": "user", "content": "hi"}]}, 501), ({"prompt_token_ids": []}, 400),
                          ({"prompt_token_ids": [1], "max_tokens": 0}, 400), ({"prompt_token_ids": list(range(600))}, 400)):
            with pytest.raises(urllib.error.HTTPError) as e:
                _post(port, "/v1/chat/completions", bad)
            assert e.value.code == code
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(f"http://127.0.0.1:{port}/nope", timeout=10)
        assert e.value.code == 404
        assert srv.handle("POST", "/health", "")[0] == 405
        assert srv.requests_served >= 8
    finally:
        srv.stop()


def test_sidecar_client_and_chat_through_the_server():
    from deepseek_v4_2080ti_b200.formats import gguf as G
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with tempfile.TemporaryDirectory() as d:
        # a GGUF that only carries a tiny byte-level BPE vocabulary
        toks = [chr(c) for c in range(33, 127)] + ["Ġ", "hi", "<eos>"]
        path = os.path.join(d, "tok.gguf")
        G.write_gguf(path, {"general.architecture": "minimax-m2", "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": toks,
                            "tokenizer.ggml.merges": ["h i"], "tokenizer.ggml.token_type": [1] * (len(toks) - 1) + [3],
                            "tokenizer.ggml.eos_token_id": len(toks) - 1}, [])
        argv = [sys.executable, "-m", "pocketllm.sidecar", "--gguf", path]
        env_backup = os.environ.get("PYTHONPATH")
        os.environ["PYTHONPATH"] = root + (os.pathsep + env_backup if env_backup else "")
        try:
            sc = cpp.PythonSidecar(argv, 30000)
            assert sc.ping() and sc.running
            enc = json.loads(sc.call(json.dumps({"op": "encode", "family": "minimax_m2", "messages": [{"role": "user", "content": "hi"}]})))
            assert enc["ok"] and enc["token_ids"] and "hi" in enc["prompt"]
            assert not json.loads(sc.call(json.dumps({"op": "bogus"})))["ok"]
            sc.shutdown()
            assert not sc.running
            eng = FakeEngine()
            opt = cpp.OpenAIServerOptions()
            opt.port, opt.chat_family, opt.sidecar_argv = 0, "minimax_m2", argv
            srv = cpp.OpenAIServer(eng, opt)
            srv.start()
            try:
                st, body = _post(srv.port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4})
                out = json.loads(body)
                want = _expected(enc["token_ids"], 4)
                assert st == 200 and out["choices"][0]["token_ids"] == ([t for t in want if t != 49] if want[-1] == 49 else want)
                assert out["choices"][0]["message"]["role"] == "assistant" and isinstance(out["choices"][0]["message"]["content"], str)
                with urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/health", timeout=10) as r:
                    assert json.loads(r.read())["sidecar"] == "ok"
            finally:
                srv.stop()
        finally:
            if env_backup is None:
                os.environ.pop("PYTHONPATH", None)
            else:
                os.environ["PYTHONPATH"] = env_backup


def _raw(port, data, timeout=10.0):
    import socket
    try:
        s = socket.create_connection(("127.0.0.1", port), timeout=timeout)
    except OSError:
        return b""
    try:
        try:
            s.sendall(data)
            s.shutdown(socket.SHUT_WR)
        except OSError:                                     # the server may answer and close before the body is out
            pass
        out = b""
        while True:
            try:
                c = s.recv(65536)
            except (socket.timeout, ConnectionError):
                break
            if not c:
                break
            out += c
        return out
    finally:
        s.close()


class VocabEngine(FakeEngine):
    def vocab_size(self): return 50


def test_hostile_requests_are_refused_and_the_server_keeps_serving():
    import random
    eng = VocabEngine()
    opt = cpp.OpenAIServerOptions()
    opt.port, opt.model_name = 0, "fake-model"
    srv = cpp.OpenAIServer(eng, opt)
    srv.start()
    try:
        port = srv.port
        body = json.dumps({"prompt_token_ids": [1, 2, 3], "max_tokens": 3}).encode()
        post = lambda b, length=None: (b"POST /v1/completions HTTP/1.1\r\nContent-Type: application/json\r\nContent-Length: "
                                       + str(len(b) if length is None else length).encode() + b"\r\n\r\n" + b)
        status = lambda raw: int(raw.split(b" ", 2)[1]) if raw.startswith(b"HTTP/1.1 ") else None
        assert status(_raw(port, post(body))) == 200
        # lengths that are not plain digits are refused rather than guessed
        for length in ("-5", "abc", "12x", ""):
            assert status(_raw(port, post(body, length))) == 400, length
        assert status(_raw(port, post(body, "99999999999999999999"))) == 413
        assert status(_raw(port, b"GET /health HTTP/1.1\r\nX: " + b"a" * 2_000_000 + b"\r\n\r\n")) == 413
        assert _raw(port, post(body, 100000)) == b""                       # the body never arrives: no answer, no thread left behind
        assert status(_raw(port, b"GET /health\r\n\r\n")) == 400
        assert _raw(port, os.urandom(300)) in (b"",) or True
        # token ids: whole numbers inside the vocabulary only - a kernel would index a table with them
        for ids in ([1.5], [-3], [1e30], ["7"], [None], [50], [2 ** 31], "12", {"a": 1}):
            raw = _raw(port, post(json.dumps({"prompt_token_ids": ids, "max_tokens": 2}).encode()))
            assert status(raw) == 400 and b"invalid_request_error" in raw, ids
        assert status(_raw(port, post(json.dumps({"prompt_token_ids": [49, 0, 7.0], "max_tokens": 2}).encode()))) == 200
        for b in (b"{{{{{", b"[" * 100001 + b"]" * 100001, b'{"prompt_token_ids":[1],"max_tokens":1e18}', b'{"prompt_token_ids":[1],"max_tokens":"y"}'):
            assert status(_raw(port, post(b))) == 400
        # random byte damage to a valid request, idle connections, then a normal request still works
        rng = random.Random(5)
        good = post(body)
        for _ in range(100):
            b = bytearray(good)
            for _ in range(rng.randrange(1, 8)):
                b[rng.randrange(len(b))] = rng.randrange(256)
            _raw(port, bytes(b), timeout=1.0)
        import socket
        idle = [socket.create_connection(("127.0.0.1", port)) for _ in range(16)]
        assert status(_raw(port, good)) == 200
        for s in idle:
            s.close()
    finally:
        srv.stop()


def test_an_engine_that_does_not_know_its_vocabulary_still_gets_whole_non_negative_ids():
    eng = FakeEngine()
    assert cpp.InferenceEngine.vocab_size(eng) == 0
    opt = cpp.OpenAIServerOptions()
    opt.port = 0
    srv = cpp.OpenAIServer(eng, opt)
    assert srv.handle("POST", "/v1/completions", json.dumps({"prompt_token_ids": [-1], "max_tokens": 1}))[0] == 400
    assert srv.handle("POST", "/v1/completions", json.dumps({"prompt_token_ids": [0.5], "max_tokens": 1}))[0] == 400
