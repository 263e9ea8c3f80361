"""PocketLLM on B200: the user-facing API (``EngineArgs``, ``LLM``, ``AsyncLLM``, ``pocketllm serve``)
over the sm_100a native engine in ``deepseek_v4_2080ti_b200``.  Importing this package does not import torch."""
from .api import (BackendCapabilities, BackendUnavailableError, ConfigurationError, EngineArgs, EngineBackend,
                  GenerationRequest, GenerationResult, HealthStatus, PocketLLMError, RequestCancelledError,
                  SamplingParams, TensorParallelSupervisorError, TimingMetrics, TokenEvent,
                  UnsupportedFeatureError, Usage)

__version__ = "0.1.0"


def __getattr__(name: str):
    if name in ("LLM", "AsyncLLM"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)


__all__ = ["AsyncLLM", "BackendCapabilities", "BackendUnavailableError", "ConfigurationError", "EngineArgs",
           "EngineBackend", "GenerationRequest", "GenerationResult", "HealthStatus", "LLM", "PocketLLMError",
           "RequestCancelledError", "SamplingParams", "TensorParallelSupervisorError", "TimingMetrics",
           "TokenEvent", "UnsupportedFeatureError", "Usage"]
