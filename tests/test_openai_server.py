"""OpenAI-compatible server against a fake backend: routes, SSE, error mapping, metrics, cancel."""
import http.client
import json
import threading

import pytest

from pocketllm import EngineArgs
from pocketllm.backends.native_backend import NativeBackend
from pocketllm.server.metrics import Metrics
from pocketllm.server.openai import error_status, make_server
from tests.test_public_api import FakeRuntime


@pytest.fixture()
def server():
    backend = NativeBackend(EngineArgs(model="fake"), runtime=FakeRuntime())
    httpd, state = make_server(backend, "127.0.0.1", 0, "fake-model")
    t = threading.Thread(target=httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True)
    t.start()
    yield httpd.server_address[1], state
    httpd.shutdown()
    httpd.server_close()


def call(port, method, path, body=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    data = None if body is None else json.dumps(body)
    c.request(method, path, body=data, headers={"Content-Type": "application/json"} if data else {})
    r = c.getresponse()
    raw = r.read()
    c.close()
    return r.status, raw


def test_health_models_metrics(server):
    port, _ = server
    st, raw = call(port, "GET", "/health")
    assert st == 200 and json.loads(raw)["ready"] is True
    assert call(port, "GET", "/ready")[0] == 200 and call(port, "GET", "/alive")[0] == 200
    st, raw = call(port, "GET", "/v1/models")
    assert json.loads(raw)["data"][0]["id"] == "fake-model"
    assert call(port, "GET", "/nope")[0] == 404
    st, raw = call(port, "GET", "/metrics")
    assert st == 200 and b"pocketllm_requests_in_flight" in raw


def test_completion_and_chat(server):
    port, _ = server
    st, raw = call(port, "POST", "/v1/completions", {"prompt": "A", "max_tokens": 3})
    body = json.loads(raw)
    assert st == 200 and body["choices"][0]["text"] == "BCD" and body["usage"]["completion_tokens"] == 3
    assert "prefill_tps" in body["timings"]
    st, raw = call(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 2})
    body = json.loads(raw)
    assert st == 200 and body["object"] == "chat.completion" and body["choices"][0]["message"]["role"] == "assistant"
    st, raw = call(port, "GET", "/metrics")
    assert b'pocketllm_requests_total{route="/v1/completions"} 1' in raw


def test_error_mapping(server):
    port, _ = server
    assert call(port, "POST", "/v1/completions", {"prompt": ""})[0] == 400
    assert call(port, "POST", "/v1/completions", {"prompt": "A", "temperature": 0.9})[0] == 501
    st, raw = call(port, "POST", "/v1/chat/completions", {"messages": []})
    assert st == 400 and json.loads(raw)["error"]["type"] == "invalid_request_error"
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request("POST", "/v1/completions", body="{not json", headers={"Content-Type": "application/json"})
    assert c.getresponse().status == 400
    from pocketllm import BackendUnavailableError, RequestCancelledError
    assert error_status(BackendUnavailableError("x")) == 503 and error_status(RequestCancelledError("x")) == 499
    assert error_status(RuntimeError("x")) == 500


def test_sse_stream(server):
    port, _ = server
    st, raw = call(port, "POST", "/v1/chat/completions",
                   {"messages": [{"role": "user", "content": "x"}], "max_tokens": 3, "stream": True})
    assert st == 200
    events = [l[6:] for l in raw.decode().split("\n\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    assert len(text) == 3
    assert chunks[-1]["choices"][0]["finish_reason"] == "length" and chunks[-1]["usage"]["completion_tokens"] == 3


def test_cancel_unknown_request_and_options(server):
    port, _ = server
    st, raw = call(port, "DELETE", "/v1/requests/nope")
    assert st == 404 and json.loads(raw)["cancelled"] is False
    assert call(port, "OPTIONS", "/v1/chat/completions")[0] == 204


def test_metrics_registry_quantiles():
    m = Metrics()
    for v in range(1, 101):
        m.observe("lat", float(v))
    m.inc("n", labels={"a": 'x"y'})
    text = m.render()
    assert 'pocketllm_lat{quantile="0.5"} 50.5' in text and "pocketllm_lat_count 100" in text
    assert 'a="x\\"y"' in text


def test_batched_serving_groups_concurrent_requests(monkeypatch):
    monkeypatch.setenv("POCKETLLM_SERVING_BATCH_WAIT_MS", "300")
    backend = NativeBackend(EngineArgs(model="fake"), runtime=FakeRuntime())
    sizes = []
    inner = backend.generate

    def spy(reqs):
        reqs = list(reqs)
        sizes.append(len(reqs))
        return inner(reqs)
    backend.generate = spy
    httpd, state = make_server(backend, "127.0.0.1", 0, "fake-model", batch_requests=True)
    t = threading.Thread(target=httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True)
    t.start()
    try:
        port, out = httpd.server_address[1], [None] * 3
        ts = [threading.Thread(target=lambda i=i: out.__setitem__(i, call(port, "POST", "/v1/completions",
                                                                          {"prompt": "A", "max_tokens": 3}))) for i in range(3)]
        for x in ts:
            x.start()
        for x in ts:
            x.join()
        assert all(st == 200 and json.loads(raw)["choices"][0]["text"] == "BCD" for st, raw in out)
        assert sum(sizes) == 3 and max(sizes) >= 2 and state.batching.stats.batched_requests == 3
    finally:
        httpd.shutdown()
        httpd.server_close()
        state.batching.close()


def test_n_choices_in_one_response_and_not_in_a_stream(server):
    port, _ = server
    st, raw = call(port, "POST", "/v1/completions", {"prompt": "A", "max_tokens": 3, "n": 3})
    body = json.loads(raw)
    assert st == 200 and [c["index"] for c in body["choices"]] == [0, 1, 2]
    assert all(c["text"] == "BCD" for c in body["choices"])                  # greedy: the choices coincide
    assert (body["usage"]["prompt_tokens"], body["usage"]["completion_tokens"], body["usage"]["total_tokens"]) == (1, 9, 10)
    st, raw = call(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 2, "n": 2})
    body = json.loads(raw)
    assert st == 200 and len(body["choices"]) == 2 and body["choices"][1]["message"]["role"] == "assistant"
    st, raw = call(port, "POST", "/v1/completions", {"prompt": "A", "max_tokens": 3, "n": 2, "stream": True})
    assert st in (400, 501) and b"n must be 1" in raw
    st, raw = call(port, "POST", "/v1/completions", {"prompt": "A", "n": 99})
    assert st == 400


def test_malformed_bodies_are_client_errors(server):
    import socket
    port, _ = server

    def raw(data):
        s = socket.create_connection(("127.0.0.1", port), timeout=20)
        try:
            try:
                s.sendall(data)
                s.shutdown(socket.SHUT_WR)
            except OSError:                                 # answered and closed before the whole body was sent
                pass
            out = b""
            while True:
                try:
                    c = s.recv(65536)
                except ConnectionError:
                    break
                if not c:
                    break
                out += c
            return int(out.split(b" ", 2)[1]) if out.startswith(b"HTTP/1.") else None
        finally:
            s.close()
    body = json.dumps({"prompt": [1, 2, 3], "max_tokens": 2}).encode()
    post = lambda b, n=None: (b"POST /v1/completions HTTP/1.1\r\nContent-Type: application/json\r\nContent-Length: "
                              + str(len(b) if n is None else n).encode() + b"\r\n\r\n" + b)
    assert raw(post(body)) == 200
    for n in ("-5", "abc", "", 100000):                         # not a number; or a body that stops short of it
        assert raw(post(body, n)) == 400, n
    assert raw(post(b"[" * 100001 + b"]" * 100001)) == 400     # nesting that exhausts the parser's stack
    assert raw(post(b"{{{{")) == 400 and raw(post(b"[1, 2]")) == 400 and raw(post(b"\xff\xfe{}")) == 400
    assert raw(post(b'{"prompt": [1.5, -3], "max_tokens": 2}')) == 400
    assert raw(post(b'{"prompt": [1], "max_tokens": "y"}')) == 400
    assert raw(post(body)) == 200


def test_runtime_counters_are_exported_as_gauges(server):
    port, _ = server
    call(port, "POST", "/v1/completions", {"prompt": "A", "max_tokens": 3})
    st, raw = call(port, "GET", "/metrics")
    text = raw.decode()
    assert st == 200 and "pocketllm_runtime_requests 1" in text and "pocketllm_runtime_completion_tokens 3" in text


def test_random_byte_damage_never_takes_the_server_down(server):
    import random
    import socket
    port, _ = server
    body = json.dumps({"prompt": [1, 2, 3], "max_tokens": 2}).encode()
    good = (b"POST /v1/completions HTTP/1.1\r\nContent-Type: application/json\r\nContent-Length: " + str(len(body)).encode()
            + b"\r\n\r\n" + body)
    rng = random.Random(3)
    for _ in range(80):
        b = bytearray(good)
        for _ in range(rng.randrange(1, 8)):
            b[rng.randrange(len(b))] = rng.randrange(256)
        try:
            s = socket.create_connection(("127.0.0.1", port), timeout=5)
            s.settimeout(2)
            try:
                s.sendall(bytes(b))
                s.shutdown(socket.SHUT_WR)
                while s.recv(65536):
                    pass
            except OSError:
                pass
            finally:
                s.close()
        except OSError:
            pass
    st, raw = call(port, "POST", "/v1/completions", {"prompt": "A", "max_tokens": 2})
    assert st == 200 and json.loads(raw)["choices"][0]["text"] == "BC"


def test_idle_connections_are_dropped(monkeypatch):
    import socket
    import time
    monkeypatch.setenv("POCKETLLM_HTTP_IDLE_TIMEOUT", "1")
    backend = NativeBackend(EngineArgs(model="fake"), runtime=FakeRuntime())
    httpd, _ = make_server(backend, "127.0.0.1", 0, "fake-model")
    t = threading.Thread(target=httpd.serve_forever, kwargs={"poll_interval": 0.05}, daemon=True)
    t.start()
    try:
        port = httpd.server_address[1]
        s = socket.create_connection(("127.0.0.1", port), timeout=10)
        s.sendall(b"POST /v1/completions HTTP/1.1\r\nContent-Length: 50\r\n\r\n{")       # and then nothing
        t0 = time.time()
        data = s.recv(4096)                                   # the server gives up on the body and closes
        assert time.time() - t0 < 8 and (data == b"" or data.startswith(b"HTTP/1.1 4"))
        s.close()
        assert call(port, "POST", "/v1/completions", {"prompt": "A", "max_tokens": 1})[0] == 200
    finally:
        httpd.shutdown()
        httpd.server_close()
