"""Request batching in front of a runtime that generates for several compatible requests at once.

One worker thread owns the runtime.  It takes the oldest queued request, waits up to ``batch_wait_ms`` for others that
may share its batch (same sampling parameters, same streaming mode, whatever else ``compatible_key`` returns), stops at
``max_batch`` requests or ``max_total_tokens`` of prompt + completion budget, and hands the batch to ``run_batch``.
``run_batch(requests, emit)`` returns one result per request; while it runs it may call ``emit(i, event)`` to stream
an event to request ``i``.  Callers block in ``submit`` or iterate ``submit_stream``.

Admission happens at submit time: a full queue is a ``BackendUnavailableError`` (HTTP 503), a request that can never
fit the token budget a ``ConfigurationError`` (400).  An exception from ``run_batch`` fails that batch's requests and
the worker carries on.

Reference behaviour: DeepSeekServingEngine (src/server/engine.py:71-249: single worker, wait window, admission on the
total-token budget, batches of identical sampling options, per-request event queues).
"""
from __future__ import annotations

import os
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator, Sequence

from ..api.errors import BackendUnavailableError, ConfigurationError
from ..api.types import GenerationRequest

_END = object()


@dataclass
class BatchingStats:
    submitted: int = 0
    rejected: int = 0
    batches: int = 0
    batched_requests: int = 0
    failed_batches: int = 0
    max_batch_seen: int = 0


@dataclass
class _Pending:
    request: GenerationRequest
    stream: bool
    key: Any
    tokens: int
    done: threading.Event = field(default_factory=threading.Event)
    events: "queue.Queue[Any]" = field(default_factory=lambda: queue.Queue(maxsize=1024))
    result: Any = None
    error: BaseException | None = None


def default_key(request: GenerationRequest) -> Any:
    sp = request.sampling_params
    return tuple(sorted((k, repr(v)) for k, v in vars(sp).items()))


def request_tokens(request: GenerationRequest) -> int:
    """Prompt length (tokens when given, else a 4-characters-per-token estimate) plus the completion budget."""
    n = len(request.prompt_tokens) if request.prompt_tokens is not None else (len(request.prompt or "") + 3) // 4
    return n + int(getattr(request.sampling_params, "max_tokens", 0) or 0)


class BatchingQueue:
    def __init__(self, run_batch: Callable[[Sequence[GenerationRequest], Callable[[int, Any], None]], Sequence[Any]],
                 max_queue: int = 32, max_batch: int = 8, batch_wait_ms: float = 2.0, max_total_tokens: int = 0,
                 compatible_key: Callable[[GenerationRequest], Any] = default_key):
        self._run_batch, self._key = run_batch, compatible_key
        self.max_queue, self.max_batch = int(max_queue), max(1, int(max_batch))
        self.batch_wait_s, self.max_total_tokens = max(0.0, batch_wait_ms) / 1e3, int(max_total_tokens)
        self.stats = BatchingStats()
        self._cv = threading.Condition()
        self._pending: list[_Pending] = []
        self._closed = False
        self._worker = threading.Thread(target=self._loop, name="pocketllm-batching", daemon=True)
        self._worker.start()

    @classmethod
    def from_env(cls, run_batch, prefix: str = "POCKETLLM_SERVING", **kw) -> "BatchingQueue":
        """``<prefix>_MAX_QUEUE``, ``_MAX_BATCH``, ``_BATCH_WAIT_MS`` and ``_MAX_TOTAL_TOKENS`` override the defaults."""
        env = lambda name, default: type(default)(os.environ.get(f"{prefix}_{name}", default))
        return cls(run_batch, max_queue=env("MAX_QUEUE", 32), max_batch=env("MAX_BATCH", 8),
                   batch_wait_ms=env("BATCH_WAIT_MS", 2.0), max_total_tokens=env("MAX_TOTAL_TOKENS", 0), **kw)

    # ---- callers
    def _enqueue(self, request: GenerationRequest, stream: bool) -> _Pending:
        tokens = request_tokens(request)
        if self.max_total_tokens and tokens > self.max_total_tokens:
            self.stats.rejected += 1
            raise ConfigurationError(f"request needs {tokens} tokens, the serving budget is {self.max_total_tokens}")
        p = _Pending(request, stream, (stream, self._key(request)), tokens)
        with self._cv:
            if self._closed:
                raise BackendUnavailableError("the batching queue is closed")
            if len(self._pending) >= self.max_queue:
                self.stats.rejected += 1
                raise BackendUnavailableError(f"serving queue is full ({self.max_queue} requests waiting)")
            self._pending.append(p)
            self.stats.submitted += 1
            self._cv.notify_all()
        return p

    def submit(self, request: GenerationRequest, timeout: float | None = None) -> Any:
        p = self._enqueue(request, False)
        if not p.done.wait(timeout):
            raise TimeoutError(f"request {request.request_id} did not finish in {timeout} s")
        if p.error is not None:
            raise p.error
        return p.result

    def submit_stream(self, request: GenerationRequest) -> Iterator[Any]:
        """Events of the request as ``run_batch`` emits them; the final result is the generator's return value."""
        p = self._enqueue(request, True)
        while True:
            ev = p.events.get()
            if ev is _END:
                break
            yield ev
        if p.error is not None:
            raise p.error
        return p.result

    def close(self, timeout: float = 5.0) -> None:
        with self._cv:
            self._closed = True
            waiting, self._pending = self._pending, []
            self._cv.notify_all()
        for p in waiting:
            self._finish(p, None, BackendUnavailableError("the batching queue was closed"))
        self._worker.join(timeout)

    # ---- worker
    def _finish(self, p: _Pending, result: Any, error: BaseException | None) -> None:
        p.result, p.error = result, error
        p.events.put(_END)
        p.done.set()

    def _collect(self) -> list[_Pending] | None:
        with self._cv:
            while not self._pending and not self._closed:
                self._cv.wait()
            if self._closed:
                return None
            first = self._pending.pop(0)
            batch, tokens = [first], first.tokens
            deadline = time.monotonic() + self.batch_wait_s
            while len(batch) < self.max_batch:
                took = False
                for i, c in enumerate(self._pending):
                    fits = not self.max_total_tokens or tokens + c.tokens <= self.max_total_tokens
                    if c.key == first.key and fits:
                        batch.append(self._pending.pop(i))
                        tokens += c.tokens
                        took = True
                        break
                if took:
                    continue
                left = deadline - time.monotonic()
                if left <= 0 or self._closed:
                    break
                self._cv.wait(left)
            return batch

    def _loop(self) -> None:
        while True:
            batch = self._collect()
            if batch is None:
                return
            self.stats.batches += 1
            self.stats.batched_requests += len(batch)
            self.stats.max_batch_seen = max(self.stats.max_batch_seen, len(batch))

            def emit(i: int, event: Any, _b=batch) -> None:
                if _b[i].stream:
                    _b[i].events.put(event)

            try:
                results = self._run_batch([p.request for p in batch], emit)
                if len(results) != len(batch):
                    raise RuntimeError(f"run_batch returned {len(results)} results for {len(batch)} requests")
                for p, r in zip(batch, results):
                    self._finish(p, r, None)
            except BaseException as exc:  # noqa: BLE001 - the worker must survive a failing batch
                self.stats.failed_batches += 1
                for p in batch:
                    self._finish(p, None, exc)
