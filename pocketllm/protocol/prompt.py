"""Chat prompt -> token ids.  Two routes: a Hugging Face ``chat_template`` shipped with the
checkpoint's tokenizer, or one of this repo's model-family encoders (DeepSeek / GLM / MiniMax
style) from ``deepseek_v4_2080ti_b200.encoding``.  Heavy imports are lazy
(reference surface: pocketllm/protocol/prompt.py:94-221)."""
from __future__ import annotations

from typing import Any

from ..api.errors import ConfigurationError
from .chat import ChatRequest, fallback_prompt


class TokenizerHandle:
    """Uniform ``encode`` / ``decode`` over a HF tokenizer, a GGUF-metadata BPE tokenizer, or a byte fallback."""

    def __init__(self, impl: Any, kind: str):
        self.impl, self.kind = impl, kind

    @classmethod
    def load(cls, path: str | None) -> "TokenizerHandle":
        if not path:
            return cls(None, "bytes")
        import os
        if os.path.isfile(path) and path.endswith(".gguf"):
            from deepseek_v4_2080ti_b200.encoding.gguf_tokenizer import GGUFTokenizer
            return cls(GGUFTokenizer.from_gguf(path), "gguf")
        if os.path.isdir(path) and os.path.exists(os.path.join(path, "tokenizer.json")) or \
                os.path.exists(os.path.join(path, "tokenizer_config.json")):
            try:
                from transformers import AutoTokenizer
                return cls(AutoTokenizer.from_pretrained(path, trust_remote_code=False), "hf")
            except Exception as exc:  # pragma: no cover - depends on the checkpoint
                raise ConfigurationError(f"cannot load tokenizer from {path}: {exc}") from exc
        return cls(None, "bytes")

    @property
    def eos_token_id(self) -> int | None:
        if self.kind == "hf":
            return self.impl.eos_token_id
        if self.kind == "gguf":
            return self.impl.eos_id
        return None

    @property
    def has_chat_template(self) -> bool:
        return self.kind == "hf" and bool(getattr(self.impl, "chat_template", None))

    def encode(self, text: str) -> list[int]:
        if self.kind == "hf":
            return list(self.impl.encode(text, add_special_tokens=False))
        if self.kind == "gguf":
            return self.impl.encode(text)
        return list(text.encode("utf-8"))

    def decode(self, ids: list[int]) -> str:
        if self.kind == "hf":
            return self.impl.decode(ids, skip_special_tokens=True)
        if self.kind == "gguf":
            return self.impl.decode(ids)
        return bytes(i & 0xFF for i in ids).decode("utf-8", errors="replace")


def _encode_with_template(tok: TokenizerHandle, chat: ChatRequest) -> list[int]:
    kwargs: dict[str, Any] = {"add_generation_prompt": chat.add_generation_prompt, "tokenize": True}
    if chat.tools:
        kwargs["tools"] = chat.tools
    try:
        ids = tok.impl.apply_chat_template(chat.messages_with_instruction(), enable_thinking=chat.thinking, **kwargs)
    except TypeError:
        ids = tok.impl.apply_chat_template(chat.messages_with_instruction(), **kwargs)
    if hasattr(ids, "input_ids"):
        ids = ids["input_ids"]
    return [int(i) for i in ids]


def _encode_with_family(tok: TokenizerHandle, chat: ChatRequest, family: str) -> list[int]:
    from deepseek_v4_2080ti_b200 import encoding
    text = encoding.render_chat(family, chat.messages_with_instruction(family == "deepseek_v4"), tools=chat.tools, thinking=chat.thinking,
                                reasoning_effort=chat.reasoning_effort,
                                add_generation_prompt=chat.add_generation_prompt)
    return tok.encode(text)


def encode_chat_prompt(tok: TokenizerHandle, chat: ChatRequest, family: str | None = None) -> list[int]:
    """Token ids for a chat request. ``family``: deepseek_v4 | glm_dsa | minimax_m2 | None (template or fallback)."""
    if family:
        return _encode_with_family(tok, chat, family)
    if tok.has_chat_template:
        return _encode_with_template(tok, chat)
    return tok.encode(fallback_prompt(chat.messages_with_instruction(), chat.add_generation_prompt))
