"""``LLM`` and ``AsyncLLM``: the synchronous and asyncio facades over one engine backend
(reference surface: pocketllm/engine.py:34-342)."""
from __future__ import annotations

import asyncio
from concurrent.futures import ThreadPoolExecutor
from typing import Any, AsyncIterator, Iterable, Iterator, Mapping, Sequence

from .api.errors import ConfigurationError
from .api.types import EngineArgs, GenerationRequest, GenerationResult, SamplingParams, TokenEvent
from .backends.factory import create_backend


def _as_args(model: str | EngineArgs | None, kw: dict[str, Any]) -> EngineArgs:
    if isinstance(model, EngineArgs):
        if kw:
            raise ConfigurationError("pass either an EngineArgs object or keyword arguments, not both")
        return model
    return EngineArgs(model=model or "", **kw)


def _as_requests(prompts: Any, sampling_params: SamplingParams | Sequence[SamplingParams] | None) -> list[GenerationRequest]:
    if isinstance(prompts, (str, GenerationRequest)) or (isinstance(prompts, Sequence) and prompts and isinstance(prompts[0], int)):
        prompts = [prompts]
    prompts = list(prompts)
    if isinstance(sampling_params, SamplingParams) or sampling_params is None:
        sps = [sampling_params or SamplingParams()] * len(prompts)
    else:
        sps = list(sampling_params)
        if len(sps) != len(prompts):
            raise ConfigurationError("sampling_params must match the number of prompts")
    out = []
    for p, sp in zip(prompts, sps):
        if isinstance(p, GenerationRequest):
            out.append(p)
        elif isinstance(p, str):
            out.append(GenerationRequest(prompt=p, sampling_params=sp))
        elif isinstance(p, Mapping) and "prompt_token_ids" in p:
            out.append(GenerationRequest(prompt_tokens=list(p["prompt_token_ids"]), sampling_params=sp))
        else:
            out.append(GenerationRequest(prompt_tokens=list(p), sampling_params=sp))
    return out


class LLM:
    """Blocking engine facade.

        llm = LLM("/ckpt/qwen", tensor_parallel_size=8)
        print(llm.generate("hello", SamplingParams(max_tokens=32))[0].text)
    """

    def __init__(self, model: str | EngineArgs | None = None, *, backend: Any = None, **kwargs: Any):
        self.args = _as_args(model, kwargs) if backend is None or model is not None else EngineArgs()
        self.backend = backend if backend is not None else create_backend(self.args)

    # ---- generation
    def generate(self, prompts: Any, sampling_params: SamplingParams | Sequence[SamplingParams] | None = None) -> list[GenerationResult]:
        return self.backend.generate(_as_requests(prompts, sampling_params))

    def generate_stream(self, prompt: Any, sampling_params: SamplingParams | None = None) -> Iterator[TokenEvent]:
        (req,) = _as_requests(prompt, sampling_params)
        return self.backend.stream(req)

    # ---- chat
    def _chat_request(self, messages: Sequence[Mapping[str, Any]], sampling_params: SamplingParams | None,
                      **body: Any) -> GenerationRequest:
        from .protocol.requests import build_chat_request
        self.backend.prepare()
        payload = {"messages": list(messages), **body}
        req, _ = build_chat_request(payload, self.backend.tokenizer, getattr(self.backend, "family", None))
        if sampling_params is not None:
            req.sampling_params = sampling_params
        return req

    def chat(self, messages: Sequence[Mapping[str, Any]], sampling_params: SamplingParams | None = None, **body: Any) -> GenerationResult:
        return self.backend.generate([self._chat_request(messages, sampling_params, **body)])[0]

    def chat_stream(self, messages: Sequence[Mapping[str, Any]], sampling_params: SamplingParams | None = None,
                    **body: Any) -> Iterator[TokenEvent]:
        return self.backend.stream(self._chat_request(messages, sampling_params, **body))

    # ---- control
    def cancel(self, request_id: str) -> bool:
        return self.backend.cancel(request_id)

    def health(self):
        return self.backend.health()

    def close(self) -> None:
        self.backend.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


class AsyncLLM:
    """asyncio mirror of ``LLM``: every blocking call runs on a private thread pool."""

    def __init__(self, model: str | EngineArgs | None = None, *, backend: Any = None, max_workers: int = 4, **kwargs: Any):
        self._llm = LLM(model, backend=backend, **kwargs)
        self._pool = ThreadPoolExecutor(max_workers=max_workers, thread_name_prefix="pocketllm-async")

    @property
    def backend(self):
        return self._llm.backend

    async def _call(self, fn, *a, **k):
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(self._pool, lambda: fn(*a, **k))

    async def generate(self, prompts: Any, sampling_params=None) -> list[GenerationResult]:
        return await self._call(self._llm.generate, prompts, sampling_params)

    async def chat(self, messages, sampling_params=None, **body) -> GenerationResult:
        return await self._call(self._llm.chat, messages, sampling_params, **body)

    async def _aiter(self, make_iter) -> AsyncIterator[TokenEvent]:
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        done = object()

        def pump() -> None:
            try:
                for ev in make_iter():
                    loop.call_soon_threadsafe(q.put_nowait, ev)
            except BaseException as exc:
                loop.call_soon_threadsafe(q.put_nowait, exc)
            finally:
                loop.call_soon_threadsafe(q.put_nowait, done)

        self._pool.submit(pump)
        while True:
            item = await q.get()
            if item is done:
                return
            if isinstance(item, BaseException):
                raise item
            yield item

    def generate_stream(self, prompt: Any, sampling_params=None) -> AsyncIterator[TokenEvent]:
        return self._aiter(lambda: self._llm.generate_stream(prompt, sampling_params))

    def chat_stream(self, messages, sampling_params=None, **body) -> AsyncIterator[TokenEvent]:
        return self._aiter(lambda: self._llm.chat_stream(messages, sampling_params, **body))

    async def cancel(self, request_id: str) -> bool:
        return self._llm.cancel(request_id)

    async def close(self) -> None:
        await self._call(self._llm.close)
        self._pool.shutdown(wait=False)

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc):
        await self.close()
        return False
