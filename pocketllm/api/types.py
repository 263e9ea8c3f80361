"""Typed public API: engine arguments, sampling parameters, requests, results, events,
capabilities and health.  Field names follow the reference's surface
(pocketllm/api/types.py:52-374) so user code and the OpenAI server port over unchanged.
Nothing here imports torch.
"""
from __future__ import annotations

import os
import uuid
from dataclasses import asdict, dataclass, field
from typing import Any, Mapping

from .errors import ConfigurationError

_TRUE = {"1", "true", "yes", "on"}
_BACKENDS = {"auto", "b200", "torch", "cpp"}       # "torch" / "cpp" are accepted aliases of the single native backend
_KV_DTYPES = {"auto", "bf16", "fp16", "fp8", "turboquant_k8v4", "int8_per_token_head"}
_SPEC = {None, "mtp", "ngram", "dspark", "dflash2"}


def _env(name: str, default, cast):
    raw = os.environ.get(name)
    if raw is None or raw == "":
        return default
    if cast is bool:
        return raw.strip().lower() in _TRUE
    try:
        return cast(raw)
    except ValueError as exc:
        raise ConfigurationError(f"environment variable {name}={raw!r} is not a valid {cast.__name__}") from exc


def _stops(value: Any) -> tuple[str, ...]:
    if value is None:
        return ()
    if isinstance(value, str):
        return (value,) if value else ()
    try:
        out = tuple(str(v) for v in value if v)
    except TypeError as exc:
        raise ConfigurationError("stop must be a string or a list of strings") from exc
    if len(out) > 16:
        raise ConfigurationError("at most 16 stop strings are supported")
    return out


@dataclass
class EngineArgs:
    """Everything needed to bring up one engine (or one rank of a tensor-parallel group)."""
    model: str = ""
    backend: str = "auto"
    tokenizer_path: str | None = None
    config_path: str | None = None
    model_format: str = "auto"            # auto | safetensors | gguf | synthetic
    tensor_parallel_size: int = 1
    tensor_parallel_rank: int = 0
    device: str | int | None = None
    max_model_len: int | None = None
    dtype: str | None = None
    kv_cache_dtype: str = "auto"
    prefill_chunk_tokens: int = 0          # 0 = runtime default (8192)
    enable_prefix_caching: bool = True
    attention_window: int = 0
    attention_sink_tokens: int = 0
    speculative_method: str | None = None  # mtp | ngram (prompt lookup) | dspark | dflash2
    speculative_tokens: int = 1
    max_batch_size: int = 1
    backend_options: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.backend = (self.backend or "auto").lower()
        if self.backend not in _BACKENDS:
            raise ConfigurationError(f"unknown backend {self.backend!r}; expected one of {sorted(_BACKENDS)}")
        if self.tensor_parallel_size < 1:
            raise ConfigurationError("tensor_parallel_size must be >= 1")
        if not 0 <= self.tensor_parallel_rank < self.tensor_parallel_size:
            raise ConfigurationError("tensor_parallel_rank must lie in [0, tensor_parallel_size)")
        if self.kv_cache_dtype not in _KV_DTYPES:
            raise ConfigurationError(f"unknown kv_cache_dtype {self.kv_cache_dtype!r}")
        if self.speculative_method not in _SPEC:
            raise ConfigurationError(f"unknown speculative_method {self.speculative_method!r}")
        if self.speculative_tokens < 1 or self.speculative_tokens > 8:
            raise ConfigurationError("speculative_tokens must lie in [1, 8]")
        if self.max_batch_size < 1:
            raise ConfigurationError("max_batch_size must be >= 1")
        if self.prefill_chunk_tokens < 0 or self.attention_window < 0 or self.attention_sink_tokens < 0:
            raise ConfigurationError("prefill_chunk_tokens / attention_window / attention_sink_tokens must be >= 0")
        if self.max_model_len is not None and self.max_model_len < 1:
            raise ConfigurationError("max_model_len must be positive")
        if not isinstance(self.backend_options, dict):
            raise ConfigurationError("backend_options must be a dict")

    @property
    def checkpoint_dir(self) -> str:
        m = os.path.expanduser(self.model)
        return os.path.dirname(m) if os.path.isfile(m) else m

    @classmethod
    def from_env(cls, model: str | None = None, **overrides: Any) -> "EngineArgs":
        """Build from POCKETLLM_* variables (used by rank children spawned by the supervisor)."""
        import json

        opts_raw = os.environ.get("POCKETLLM_BACKEND_OPTIONS", "")
        try:
            opts = json.loads(opts_raw) if opts_raw else {}
        except json.JSONDecodeError as exc:
            raise ConfigurationError("POCKETLLM_BACKEND_OPTIONS is not valid JSON") from exc
        values: dict[str, Any] = dict(
            model=model or os.environ.get("POCKETLLM_CHECKPOINT", ""),
            backend=_env("POCKETLLM_BACKEND", "auto", str),
            tokenizer_path=_env("POCKETLLM_TOKENIZER", None, str),
            config_path=_env("POCKETLLM_CONFIG", None, str),
            model_format=_env("POCKETLLM_MODEL_FORMAT", "auto", str),
            tensor_parallel_size=_env("POCKETLLM_TP_SIZE", _env("WORLD_SIZE", 1, int), int),
            tensor_parallel_rank=_env("TP_RANK", _env("RANK", 0, int), int),
            device=_env("POCKETLLM_DEVICE", None, str),
            max_model_len=_env("POCKETLLM_MAX_MODEL_LEN", None, int),
            kv_cache_dtype=_env("POCKETLLM_KV_CACHE_DTYPE", "auto", str),
            prefill_chunk_tokens=_env("POCKETLLM_PREFILL_CHUNK_TOKENS", 0, int),
            enable_prefix_caching=_env("POCKETLLM_PREFIX_CACHING", True, bool),
            max_batch_size=_env("POCKETLLM_MAX_BATCH_SIZE", 1, int),
            speculative_method=_env("POCKETLLM_SPECULATIVE_METHOD", None, str),
            speculative_tokens=_env("POCKETLLM_SPECULATIVE_TOKENS", 1, int),
            backend_options=opts,
        )
        values.update(overrides)
        return cls(**values)


MAX_CHOICES = 16


@dataclass
class SamplingParams:
    max_tokens: int = 256
    temperature: float = 0.0
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    seed: int | None = None
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    stop: tuple[str, ...] = ()
    n: int = 1
    logprobs: bool = False
    top_logprobs: int | None = None
    response_format: dict[str, Any] | None = None
    extra: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.stop = _stops(self.stop)
        if self.max_tokens < 1:
            raise ConfigurationError("max_tokens must be >= 1")
        if self.temperature < 0:
            raise ConfigurationError("temperature must be >= 0")
        if self.top_p is not None and not 0 < self.top_p <= 1:
            raise ConfigurationError("top_p must lie in (0, 1]")
        if self.top_k is not None and self.top_k < 0:
            raise ConfigurationError("top_k must be >= 0")
        if self.min_p is not None and not 0 <= self.min_p <= 1:
            raise ConfigurationError("min_p must lie in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ConfigurationError("repetition_penalty must be > 0")
        if not 1 <= self.n <= MAX_CHOICES:
            raise ConfigurationError(f"n must lie in [1, {MAX_CHOICES}]")
        if self.top_logprobs is not None and not 0 <= self.top_logprobs <= 20:
            raise ConfigurationError("top_logprobs must lie in [0, 20]")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 1e-5

    @classmethod
    def from_openai(cls, body: Mapping[str, Any]) -> "SamplingParams":
        def pick(*names, default=None):
            for n in names:
                if body.get(n) is not None:
                    return body[n]
            return default

        try:
            return cls(
                max_tokens=int(pick("max_completion_tokens", "max_tokens", default=256)),
                temperature=float(pick("temperature", default=0.0)),
                top_p=None if pick("top_p") is None else float(pick("top_p")),
                top_k=None if pick("top_k") is None else int(pick("top_k")),
                min_p=None if pick("min_p") is None else float(pick("min_p")),
                seed=None if pick("seed") is None else int(pick("seed")),
                repetition_penalty=float(pick("repetition_penalty", default=1.0)),
                frequency_penalty=float(pick("frequency_penalty", default=0.0)),
                presence_penalty=float(pick("presence_penalty", default=0.0)),
                stop=_stops(pick("stop")),
                n=int(pick("n", default=1)),
                logprobs=bool(pick("logprobs", default=False)),
                # the completions API gives the number of alternatives as an integer "logprobs"; chat uses "top_logprobs"
                top_logprobs=int(pick("top_logprobs")) if pick("top_logprobs") is not None else
                (int(pick("logprobs")) if isinstance(pick("logprobs"), int) and not isinstance(pick("logprobs"), bool) else None),
                response_format=pick("response_format"),
            )
        except (TypeError, ValueError) as exc:
            if isinstance(exc, ConfigurationError):
                raise
            raise ConfigurationError(f"invalid sampling parameter: {exc}") from exc

    def to_generation_options(self) -> dict[str, Any]:
        d = asdict(self)
        d["stop"] = list(self.stop)
        d["greedy"] = self.greedy
        return d


@dataclass
class Usage:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0

    @property
    def total_tokens(self) -> int:
        return self.prompt_tokens + self.completion_tokens

    def as_dict(self) -> dict[str, int]:
        return {"prompt_tokens": self.prompt_tokens, "completion_tokens": self.completion_tokens,
                "total_tokens": self.total_tokens,
                "prompt_tokens_details": {"cached_tokens": self.cached_tokens}}


@dataclass
class TimingMetrics:
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    total_seconds: float = 0.0
    ttft_seconds: float = 0.0
    tpot_seconds: float = 0.0

    @classmethod
    def from_mapping(cls, values: Mapping[str, Any] | None) -> "TimingMetrics":
        values = values or {}
        return cls(**{k: float(values.get(k, 0.0) or 0.0) for k in cls.__dataclass_fields__})

    def throughput(self, usage: "Usage") -> dict[str, float]:
        """prefill_tps counts the first generated token in prefill (docs/benchmarking.md:21-32 of the reference)."""
        pre = usage.prompt_tokens / self.prefill_seconds if self.prefill_seconds > 0 else 0.0
        dec_tokens = max(0, usage.completion_tokens - 1)
        dec = dec_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0
        return {"prefill_tps": pre, "decode_tps": dec}

    def as_dict(self) -> dict[str, float]:
        return asdict(self)


@dataclass
class GenerationRequest:
    prompt: str | None = None
    prompt_tokens: list[int] | None = None
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    request_id: str = field(default_factory=lambda: f"req-{uuid.uuid4().hex}")
    metadata: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.prompt is None and self.prompt_tokens is None:
            raise ConfigurationError("a request needs either prompt text or prompt_tokens")
        if self.prompt_tokens is not None:
            try:
                self.prompt_tokens = [int(t) for t in self.prompt_tokens]
            except (TypeError, ValueError) as exc:
                raise ConfigurationError("prompt_tokens must be integers") from exc
            if not self.prompt_tokens:
                raise ConfigurationError("prompt_tokens must not be empty")
            if min(self.prompt_tokens) < 0:
                raise ConfigurationError("prompt_tokens must be non-negative")


@dataclass
class GenerationResult:
    request_id: str
    token_ids: list[int] = field(default_factory=list)
    text: str = ""
    finish_reason: str = "stop"
    usage: Usage = field(default_factory=Usage)
    timings: TimingMetrics = field(default_factory=TimingMetrics)
    logprobs: Any = None
    metadata: dict[str, Any] = field(default_factory=dict)
    choices: list["GenerationResult"] = field(default_factory=list)      # all n completions when n > 1 (this one is choices[0])


@dataclass
class TokenEvent:
    request_id: str
    token_id: int | None = None
    text: str = ""
    finish_reason: str | None = None
    usage: Usage | None = None
    metadata: dict[str, Any] = field(default_factory=dict)


@dataclass
class BackendCapabilities:
    name: str
    models: tuple[str, ...] = ()
    model_formats: tuple[str, ...] = ()
    devices: tuple[str, ...] = ()
    supports_batch: bool = False
    supports_streaming: bool = True
    supports_cancellation: bool = False
    supports_embeddings: bool = False
    supports_logprobs: bool = False
    supports_structured_outputs: bool = False
    supports_prefix_caching: bool = False
    supports_speculative_decoding: tuple[str, ...] = ()
    details: dict[str, Any] = field(default_factory=dict)

    def supports(self, feature: str) -> bool:
        if feature.startswith("speculative:"):
            return feature.split(":", 1)[1] in self.supports_speculative_decoding
        return bool(getattr(self, f"supports_{feature}", False))


@dataclass
class HealthStatus:
    status: str                 # ok | loading | error | closed
    backend: str
    ready: bool
    message: str = ""
    details: dict[str, Any] = field(default_factory=dict)

    @property
    def alive(self) -> bool:
        return self.status in ("ok", "loading")

    def as_dict(self) -> dict[str, Any]:
        return {"status": self.status, "backend": self.backend, "ready": self.ready, "alive": self.alive,
                "message": self.message, "details": self.details}
