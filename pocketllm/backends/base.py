"""Shared bookkeeping for backends: a re-entrant lock, open/closed state, and the cancel set
(reference surface: pocketllm/backends/base.py:20-117)."""
from __future__ import annotations

import threading
from typing import Iterable, Iterator

from ..api.errors import BackendUnavailableError, RequestCancelledError
from ..api.types import (BackendCapabilities, EngineArgs, GenerationRequest, GenerationResult, HealthStatus,
                         TokenEvent)


class BackendBase:
    name = "base"

    def __init__(self, args: EngineArgs):
        self.args = args
        self._lock = threading.RLock()
        self._closed = False
        self._ready = False
        self._error: str | None = None
        self._cancelled: set[str] = set()
        self._active: set[str] = set()
        self._cancel_lock = threading.Lock()

    # -- lifecycle
    def _require_open(self) -> None:
        if self._closed:
            raise BackendUnavailableError(f"{self.name} backend is closed")

    def prepare(self) -> None:
        with self._lock:
            self._require_open()
            if self._ready:
                return
            try:
                self._load()
                self._ready = True
                self._error = None
            except Exception as exc:
                self._error = f"{type(exc).__name__}: {exc}"
                raise

    def _load(self) -> None:  # pragma: no cover - overridden
        raise NotImplementedError

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
            self._ready = False
            self._release()

    def _release(self) -> None:
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    # -- health
    def health(self) -> HealthStatus:
        if self._closed:
            return HealthStatus("closed", self.name, False, "backend closed")
        if self._error:
            return HealthStatus("error", self.name, False, self._error)
        if not self._ready:
            return HealthStatus("loading", self.name, False, "weights not loaded yet")
        return HealthStatus("ok", self.name, True, details=self._health_details())

    def _health_details(self) -> dict:
        return {}

    def capabilities(self) -> BackendCapabilities:  # pragma: no cover - overridden
        return BackendCapabilities(self.name)

    # -- cancellation
    def cancel(self, request_id: str) -> bool:
        with self._cancel_lock:
            if request_id in self._active:
                self._cancelled.add(request_id)
                return True
            return False

    def _begin(self, request_id: str) -> None:
        with self._cancel_lock:
            self._active.add(request_id)

    def _end(self, request_id: str) -> None:
        with self._cancel_lock:
            self._active.discard(request_id)
            self._cancelled.discard(request_id)

    def _check_cancel(self, request_id: str) -> None:
        with self._cancel_lock:
            hit = request_id in self._cancelled
        if hit:
            raise RequestCancelledError(f"request {request_id} was cancelled")

    # -- work
    def generate(self, requests: Iterable[GenerationRequest]) -> list[GenerationResult]:  # pragma: no cover
        raise NotImplementedError

    def stream(self, request: GenerationRequest) -> Iterator[TokenEvent]:  # pragma: no cover
        raise NotImplementedError

    def run_worker(self) -> None:
        raise BackendUnavailableError(f"{self.name} backend has no worker loop")
