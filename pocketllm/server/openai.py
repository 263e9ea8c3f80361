"""OpenAI-compatible HTTP server on the standard library (``ThreadingHTTPServer``).

Endpoints (same as the reference, pocketllm/server/openai.py:176-322):
  GET  /health /alive /ready /metrics /v1/models
  POST /v1/chat/completions  /v1/completions     (JSON or SSE when ``stream`` is true)
  DELETE /v1/requests/<id>                       (cancel; the request ends with HTTP 499 semantics)
  OPTIONS *                                      (CORS pre-flight)
"""
from __future__ import annotations

import json
import os
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any

from ..api.errors import (BackendUnavailableError, ConfigurationError, PocketLLMError, RequestCancelledError,
                          UnsupportedFeatureError)
from ..api.types import GenerationRequest, GenerationResult
from ..protocol.chat import extract_tool_calls, split_reasoning
from ..protocol.stream import StreamSplitter
from ..protocol.requests import build_chat_request, build_completion_request
from .metrics import Metrics

MAX_BODY = 64 << 20


def error_status(exc: BaseException) -> int:
    if isinstance(exc, (ConfigurationError, json.JSONDecodeError, KeyError, TypeError, ValueError)) and \
            not isinstance(exc, UnsupportedFeatureError):
        return 400
    if isinstance(exc, UnsupportedFeatureError):
        return 501
    if isinstance(exc, BackendUnavailableError):
        return 503
    if isinstance(exc, RequestCancelledError):
        return 499
    return 500


def error_body(exc: BaseException, status: int) -> dict[str, Any]:
    kind = {400: "invalid_request_error", 501: "not_implemented", 503: "service_unavailable", 499: "request_cancelled"}.get(status, "internal_error")
    return {"error": {"message": str(exc) or type(exc).__name__, "type": kind, "code": status}}


class ServerState:
    def __init__(self, backend: Any, served_model_name: str = "pocketllm", metrics: Metrics | None = None,
                 batching: Any = None):
        self.backend = backend
        self.batching = batching          # a BatchingQueue: non-streamed requests that arrive together share one generate call
        self.model_name = served_model_name
        self.metrics = metrics or Metrics()
        self.started = time.time()
        m = self.metrics
        m.describe("requests_total", "HTTP generation requests received")
        m.describe("request_errors_total", "generation requests that ended in an error, by type")
        m.describe("requests_in_flight", "generation requests currently being served")
        m.describe("request_latency_seconds", "end-to-end request latency")
        m.describe("time_to_first_token_seconds", "prefill latency")
        m.describe("decode_tokens_per_second", "per-request decode throughput")
        m.describe("prefill_tokens_per_second", "per-request prefill throughput")
        m.set("requests_in_flight", 0)


def _bytes(text: str) -> list[int]:
    return list(text.encode("utf-8"))


def _chat_logprobs(res: GenerationResult) -> dict[str, Any] | None:
    """OpenAI chat form: one entry per generated token with its alternatives."""
    if not res.logprobs:
        return None
    return {"content": [{"token": e["token"], "logprob": e["logprob"], "bytes": _bytes(e["token"]),
                         "top_logprobs": [{"token": a["token"], "logprob": a["logprob"], "bytes": _bytes(a["token"])}
                                          for a in e.get("top_logprobs", [])]} for e in res.logprobs]}


def _completion_logprobs(res: GenerationResult) -> dict[str, Any] | None:
    """Legacy completions form: parallel lists."""
    if not res.logprobs:
        return None
    offsets, pos = [], 0
    for e in res.logprobs:
        offsets.append(pos)
        pos += len(e["token"])
    return {"tokens": [e["token"] for e in res.logprobs], "token_logprobs": [e["logprob"] for e in res.logprobs],
            "top_logprobs": [{a["token"]: a["logprob"] for a in e.get("top_logprobs", [])} for e in res.logprobs],
            "text_offset": offsets}


def _chat_choice(index: int, res: GenerationResult, had_tools: bool) -> dict[str, Any]:
    reasoning, answer = split_reasoning(res.text)
    calls: list[dict[str, Any]] = []
    if had_tools:
        answer, calls = extract_tool_calls(answer)
    msg: dict[str, Any] = {"role": "assistant", "content": answer if (answer or not calls) else None}
    if reasoning:
        msg["reasoning_content"] = reasoning
    if calls:
        msg["tool_calls"] = calls
    return {"index": index, "message": msg, "finish_reason": "tool_calls" if calls else res.finish_reason,
            "logprobs": _chat_logprobs(res)}


def _chat_payload(state: ServerState, res: GenerationResult, created: int, had_tools: bool) -> dict[str, Any]:
    """``res.choices`` holds the n completions of a request with n > 1; usage counts the prompt once."""
    return {"id": f"chatcmpl-{res.request_id}", "object": "chat.completion", "created": created,
            "model": state.model_name,
            "choices": [_chat_choice(i, r, had_tools) for i, r in enumerate(res.choices or [res])],
            "usage": res.usage.as_dict(),
            "timings": {**res.timings.as_dict(), **res.timings.throughput(res.usage)}}


def _completion_payload(state: ServerState, res: GenerationResult, created: int) -> dict[str, Any]:
    return {"id": f"cmpl-{res.request_id}", "object": "text_completion", "created": created, "model": state.model_name,
            "choices": [{"index": i, "text": r.text, "finish_reason": r.finish_reason, "logprobs": _completion_logprobs(r)}
                        for i, r in enumerate(res.choices or [res])],
            "usage": res.usage.as_dict(),
            "timings": {**res.timings.as_dict(), **res.timings.throughput(res.usage)}}


def make_handler(state: ServerState):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "pocketllm-b200"
        # a client that connects and then says nothing (or stops reading) gives its thread back after this many seconds
        timeout = float(os.environ.get("POCKETLLM_HTTP_IDLE_TIMEOUT", "120"))

        def log_message(self, fmt, *args):  # quiet by default
            pass

        # ---- plumbing
        def _cors(self) -> None:
            self.send_header("Access-Control-Allow-Origin", "*")
            self.send_header("Access-Control-Allow-Headers", "authorization, content-type")
            self.send_header("Access-Control-Allow-Methods", "GET, POST, DELETE, OPTIONS")

        def _json(self, status: int, obj: Any) -> None:
            data = json.dumps(obj, ensure_ascii=False).encode("utf-8")
            self.send_response(status)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self._cors()
            self.end_headers()
            self.wfile.write(data)

        def _text(self, status: int, text: str, ctype: str = "text/plain; version=0.0.4") -> None:
            data = text.encode("utf-8")
            self.send_response(status)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            self._cors()
            self.end_headers()
            self.wfile.write(data)

        def _fail(self, exc: BaseException) -> None:
            status = error_status(exc)
            state.metrics.inc("request_errors_total", labels={"type": type(exc).__name__, "status": str(status)})
            try:
                self._json(status, error_body(exc, status))
            except OSError:
                pass

        def _body(self) -> dict[str, Any]:
            raw_len = (self.headers.get("Content-Length") or "").strip()
            if not raw_len.isdigit():                          # "-5", "abc", "" are refused rather than guessed
                raise ConfigurationError("Content-Length must be a whole number")
            n = int(raw_len)
            if n <= 0:
                raise ConfigurationError("request body is empty")
            if n > MAX_BODY:
                raise ConfigurationError("request body too large")
            try:
                data = self.rfile.read(n)
            except (TimeoutError, ConnectionError) as exc:     # the idle timeout: the client stopped sending
                self.close_connection = True
                raise ConfigurationError("request body did not arrive in time") from exc
            if len(data) != n:
                raise ConfigurationError("request body is shorter than its Content-Length")
            try:
                obj = json.loads(data.decode("utf-8"))
            except RecursionError as exc:                      # thousands of nested brackets
                raise ConfigurationError("request body is nested too deeply") from exc
            except ValueError as exc:                          # malformed JSON or UTF-8
                raise ConfigurationError(f"request body is not valid JSON: {exc}") from exc
            if not isinstance(obj, dict):
                raise ConfigurationError("request body must be a JSON object")
            return obj

        # ---- verbs
        def do_OPTIONS(self):
            self.send_response(204)
            self._cors()
            self.send_header("Content-Length", "0")
            self.end_headers()

        def do_GET(self):
            path = self.path.split("?", 1)[0].rstrip("/") or "/"
            try:
                if path in ("/health", "/alive", "/ready"):
                    h = state.backend.health()
                    ok = h.alive if path == "/alive" else h.ready
                    self._json(200 if ok else 503, h.as_dict())
                elif path == "/metrics":
                    state.metrics.set("uptime_seconds", time.time() - state.started)
                    # the runtime's own counters (speculation rounds / accepted drafts, prefix-cache hits, collective
                    # recoveries, swap traffic ...) as gauges named runtime_<key>
                    try:
                        details = state.backend.health().details or {}
                    except Exception:
                        details = {}
                    for k, v in details.items():
                        if isinstance(v, (int, float)) and not isinstance(v, bool):
                            state.metrics.set("runtime_" + "".join(c if c.isalnum() else "_" for c in str(k)), float(v))
                    self._text(200, state.metrics.render())
                elif path == "/v1/models":
                    self._json(200, {"object": "list", "data": [{"id": state.model_name, "object": "model",
                                                                   "created": int(state.started), "owned_by": "pocketllm"}]})
                else:
                    self._json(404, {"error": {"message": f"no route {path}", "type": "not_found", "code": 404}})
            except Exception as exc:
                self._fail(exc)

        def do_DELETE(self):
            path = self.path.split("?", 1)[0]
            if path.startswith("/v1/requests/"):
                rid = path[len("/v1/requests/"):]
                hit = state.backend.cancel(rid)
                self._json(200 if hit else 404, {"id": rid, "cancelled": bool(hit)})
            else:
                self._json(404, {"error": {"message": f"no route {path}", "type": "not_found", "code": 404}})

        def do_POST(self):
            path = self.path.split("?", 1)[0].rstrip("/")
            if path not in ("/v1/chat/completions", "/v1/completions"):
                self._json(404, {"error": {"message": f"no route {path}", "type": "not_found", "code": 404}})
                return
            m = state.metrics
            m.inc("requests_total", labels={"route": path})
            m.add("requests_in_flight", 1)
            t0 = time.time()
            try:
                body = self._body()
                rid = self.headers.get("X-Request-Id") or uuid.uuid4().hex
                state.backend.prepare()
                tok = state.backend.tokenizer
                if path.endswith("chat/completions"):
                    req, chat = build_chat_request(body, tok, getattr(state.backend, "family", None), rid)
                    had_tools = bool(chat.tools)
                    is_chat = True
                else:
                    req = build_completion_request(body, tok, rid)
                    had_tools, is_chat = False, False
                if body.get("stream"):
                    self._stream(req, is_chat, thinking=bool(is_chat and chat.thinking), tools=had_tools)
                else:
                    res = state.batching.submit(req) if state.batching is not None else state.backend.generate([req])[0]
                    created = int(t0)
                    self._json(200, _chat_payload(state, res, created, had_tools) if is_chat
                               else _completion_payload(state, res, created))
                    self._observe(res)
            except Exception as exc:
                self._fail(exc)
            finally:
                m.add("requests_in_flight", -1)
                m.observe("request_latency_seconds", time.time() - t0)

        def _observe(self, res: GenerationResult) -> None:
            m = state.metrics
            tp = res.timings.throughput(res.usage)
            if res.timings.ttft_seconds:
                m.observe("time_to_first_token_seconds", res.timings.ttft_seconds)
            if tp["decode_tps"]:
                m.observe("decode_tokens_per_second", tp["decode_tps"])
            if tp["prefill_tps"]:
                m.observe("prefill_tokens_per_second", tp["prefill_tps"])
            m.inc("prompt_tokens_total", res.usage.prompt_tokens)
            m.inc("completion_tokens_total", res.usage.completion_tokens)

        def _stream(self, req: GenerationRequest, is_chat: bool, thinking: bool = False, tools: bool = False) -> None:
            created = int(time.time())
            cid = ("chatcmpl-" if is_chat else "cmpl-") + req.request_id
            events = state.backend.stream(req)
            first = next(events, None)          # surfaces validation errors before any header is written
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.send_header("X-Request-Id", req.request_id)
            self._cors()
            self.end_headers()
            self.close_connection = True

            def emit(obj: Any) -> None:
                self.wfile.write(b"data: " + (obj if isinstance(obj, bytes) else json.dumps(obj, ensure_ascii=False).encode()) + b"\n\n")
                self.wfile.flush()

            def chunk(delta: dict[str, Any] | str, finish: str | None, usage=None) -> dict[str, Any]:
                if is_chat:
                    c = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": state.model_name,
                         "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
                else:
                    c = {"id": cid, "object": "text_completion", "created": created, "model": state.model_name,
                         "choices": [{"index": 0, "text": delta, "finish_reason": finish}]}
                if usage is not None:
                    c["usage"] = usage
                return c

            try:
                # chat streams go through the splitter: reasoning before </think>, content after it, tool-call markup
                # held out of the visible text and delivered as one tool_calls delta at the end
                split = StreamSplitter(thinking=thinking, tools=tools) if is_chat else None
                if is_chat:
                    emit(chunk({"role": "assistant", "content": ""}, None))
                ev = first
                while ev is not None:
                    if ev.text:
                        if split is None:
                            emit(chunk(ev.text, None))
                        else:
                            for d in split.feed(ev.text):
                                emit(chunk(d, None))
                    if ev.finish_reason is not None:
                        finish = ev.finish_reason
                        if split is not None:
                            tail, calls = split.finish()
                            for d in tail:
                                emit(chunk(d, None))
                            if calls:
                                emit(chunk({"tool_calls": [dict(c, index=i) for i, c in enumerate(calls)]}, None))
                                finish = "tool_calls"
                        last = chunk({} if is_chat else "", finish, ev.usage.as_dict() if ev.usage else None)
                        if ev.metadata.get("logprobs"):     # asked for with "logprobs": delivered once, with the closing chunk
                            shim = GenerationResult(req.request_id, logprobs=ev.metadata["logprobs"])
                            last["choices"][0]["logprobs"] = _chat_logprobs(shim) if is_chat else _completion_logprobs(shim)
                        emit(last)
                    ev = next(events, None)
                emit(b"[DONE]")
            except (BrokenPipeError, ConnectionResetError):
                state.backend.cancel(req.request_id)
            except Exception as exc:
                status = error_status(exc)
                state.metrics.inc("request_errors_total", labels={"type": type(exc).__name__, "status": str(status)})
                try:
                    emit(error_body(exc, status))
                    emit(b"[DONE]")
                except OSError:
                    pass

    return Handler


class _Server(ThreadingHTTPServer):
    daemon_threads = True

    def handle_error(self, request, client_address):
        """A client that went away mid-response is not an error worth a traceback; anything else is counted and shown."""
        import sys
        exc = sys.exc_info()[1]
        if isinstance(exc, (ConnectionError, TimeoutError)):
            self.client_disconnects = getattr(self, "client_disconnects", 0) + 1
            return
        super().handle_error(request, client_address)


def make_server(backend: Any, host: str = "127.0.0.1", port: int = 8000, served_model_name: str = "pocketllm",
                metrics: Metrics | None = None, batch_requests: bool | None = None) -> tuple[ThreadingHTTPServer, ServerState]:
    """``batch_requests`` (default: the ``POCKETLLM_SERVING_BATCHING`` environment switch) puts a ``BatchingQueue`` in
    front of ``backend.generate`` for non-streamed requests; its limits come from ``POCKETLLM_SERVING_*``."""
    if batch_requests is None:
        batch_requests = os.environ.get("POCKETLLM_SERVING_BATCHING", "0").lower() in ("1", "true", "yes", "on")
    batching = None
    if batch_requests:
        from .batching import BatchingQueue
        batching = BatchingQueue.from_env(lambda reqs, emit: backend.generate(list(reqs)))
    state = ServerState(backend, served_model_name, metrics, batching)
    httpd = _Server((host, port), make_handler(state))
    return httpd, state


def serve(backend: Any, host: str = "127.0.0.1", port: int = 8000, served_model_name: str = "pocketllm",
          ready_event: threading.Event | None = None) -> None:
    httpd, _ = make_server(backend, host, port, served_model_name)
    if ready_event is not None:
        ready_event.set()
    try:
        httpd.serve_forever(poll_interval=0.2)
    except KeyboardInterrupt:
        pass
    finally:
        httpd.server_close()
        backend.close()
