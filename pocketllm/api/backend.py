"""Structural interface every engine backend implements (reference: pocketllm/api/backend.py:17-45)."""
from __future__ import annotations

from typing import Iterable, Iterator, Protocol, runtime_checkable

from .types import BackendCapabilities, GenerationRequest, GenerationResult, HealthStatus, TokenEvent


@runtime_checkable
class EngineBackend(Protocol):
    def capabilities(self) -> BackendCapabilities: ...

    def health(self) -> HealthStatus: ...

    def prepare(self) -> None:
        """Load weights and warm up; idempotent."""

    def generate(self, requests: Iterable[GenerationRequest]) -> list[GenerationResult]: ...

    def stream(self, request: GenerationRequest) -> Iterator[TokenEvent]: ...

    def run_worker(self) -> None:
        """Serve commands from rank 0 until told to stop (ranks > 0 of a tensor-parallel group)."""

    def cancel(self, request_id: str) -> bool: ...

    def close(self) -> None: ...
