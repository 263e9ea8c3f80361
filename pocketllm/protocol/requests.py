"""HTTP body -> ``GenerationRequest`` for /v1/chat/completions and /v1/completions
(reference surface: pocketllm/protocol/requests.py:56-93)."""
from __future__ import annotations

from typing import Any, Mapping

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
