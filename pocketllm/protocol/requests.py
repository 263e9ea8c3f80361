"""HTTP body -> ``GenerationRequest`` for /v1/chat/completions and /v1/completions
(reference surface: pocketllm/protocol/requests.py:56-93)."""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, Mapping, Sequence

from ..api.errors import ConfigurationError
from ..api.types import GenerationRequest, SamplingParams
from .chat import ChatRequest
from .prompt import TokenizerHandle, encode_chat_prompt


def build_chat_request(body: Mapping[str, Any], tokenizer: TokenizerHandle, family: str | None = None,
                       request_id: str | None = None) -> tuple[GenerationRequest, ChatRequest]:
    chat = ChatRequest.from_body(body)
    ids = encode_chat_prompt(tokenizer, chat, family)
    if not ids:
        raise ConfigurationError("the chat prompt encoded to zero tokens")
    kw: dict[str, Any] = {}
    if request_id:
        kw["request_id"] = request_id
    req = GenerationRequest(prompt_tokens=ids, sampling_params=SamplingParams.from_openai(body),
                            metadata={"kind": "chat", "tools": bool(chat.tools), "thinking": chat.thinking,
                                      "stream": chat.stream, "model": chat.model,
                                      "response_format_in_prompt": chat.response_schema is not None}, **kw)
    return req, chat


def build_completion_request(body: Mapping[str, Any], tokenizer: TokenizerHandle,
                             request_id: str | None = None) -> GenerationRequest:
    if not isinstance(body, Mapping):
        raise ConfigurationError("request body must be a JSON object")
    prompt = body.get("prompt")
    kw: dict[str, Any] = {}
    if request_id:
        kw["request_id"] = request_id
    meta = {"kind": "completion", "stream": bool(body.get("stream", False)), "model": body.get("model")}
    params = SamplingParams.from_openai(body)
    if isinstance(prompt, str):
        if not prompt:
            raise ConfigurationError("prompt must not be empty")
        return GenerationRequest(prompt=prompt, prompt_tokens=tokenizer.encode(prompt), sampling_params=params,
                                 metadata=meta, **kw)
    if isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
        return GenerationRequest(prompt_tokens=list(prompt), sampling_params=params, metadata=meta, **kw)
    if isinstance(prompt, list) and len(prompt) == 1 and isinstance(prompt[0], str):
        return GenerationRequest(prompt=prompt[0], prompt_tokens=tokenizer.encode(prompt[0]), sampling_params=params,
                                 metadata=meta, **kw)
    raise ConfigurationError("prompt must be a string or a list of token ids")


def expand_choices(req: GenerationRequest) -> list[GenerationRequest]:
    """``n`` independent single-completion requests for a request that asks for ``n`` choices: the same prompt, ids
    ``<id>-<i>``, and - when a seed is given - seeds ``seed + i`` so that the choices differ and the whole answer stays
    reproducible (reference: the prompt is repeated ``n`` times in one batch, src/server/openai.py:364-366)."""
    sp = req.sampling_params
    if sp.n <= 1:
        return [req]
    out = []
    for i in range(sp.n):
        one = dataclasses.replace(copy.deepcopy(sp), n=1, seed=None if sp.seed is None else sp.seed + i)
        out.append(dataclasses.replace(req, sampling_params=one, request_id=f"{req.request_id}-{i}",
                                       metadata=dict(req.metadata, choice=i)))
    return out


def merge_choices(req: GenerationRequest, results: Sequence[Any]) -> Any:
    """One result for ``req`` from the results of ``expand_choices(req)``: choice 0 with ``choices`` holding all of them;
    the prompt is counted once in ``usage``, completions and time are summed."""
    if req.sampling_params.n <= 1:
        return results[0]
    from ..api.types import TimingMetrics, Usage
    first = results[0]
    usage = Usage(first.usage.prompt_tokens, sum(r.usage.completion_tokens for r in results))
    t = TimingMetrics(prefill_seconds=sum(r.timings.prefill_seconds for r in results),
                      decode_seconds=sum(r.timings.decode_seconds for r in results),
                      total_seconds=sum(r.timings.total_seconds for r in results),
                      ttft_seconds=first.timings.ttft_seconds)
    return dataclasses.replace(first, request_id=req.request_id, usage=usage, timings=t,
                               choices=[dataclasses.replace(r, choices=[]) for r in results])
