"""Chat prompt encodings per model family and the GGUF-metadata BPE tokenizer
(reference: src/encoding/deepseek_v4.py, glm_dsa.py, minimax_m2.py, gguf_tokenizer.py)."""
from __future__ import annotations

from typing import Any

from . import deepseek_v4, glm_dsa, minimax_m2  # noqa: F401

FAMILIES = ("deepseek_v4", "glm_dsa", "minimax_m2")


def render_chat(family: str, messages: list[dict[str, Any]], tools: list[dict] | None = None, thinking: bool = False,
                reasoning_effort: str | None = None, add_generation_prompt: bool = True) -> str:
    """Prompt text for a conversation in the family's native chat format."""
    if family == "deepseek_v4":
        return deepseek_v4.render(messages, tools=tools, thinking=thinking, reasoning_effort=reasoning_effort,
                                  add_generation_prompt=add_generation_prompt)
    if family == "glm_dsa":
        return glm_dsa.render(messages, tools=tools, thinking=thinking, add_generation_prompt=add_generation_prompt)
    if family == "minimax_m2":
        return minimax_m2.render(messages, tools=tools, thinking=thinking, add_generation_prompt=add_generation_prompt)
    raise ValueError(f"unknown chat family {family!r} (expected one of {FAMILIES})")


def parse_completion(family: str, text: str, thinking: bool = False) -> dict[str, Any]:
    """Split a completion into ``content``, ``reasoning_content`` and OpenAI-style ``tool_calls``."""
    if family == "deepseek_v4":
        return deepseek_v4.parse_completion(text, thinking)
    if family in ("glm_dsa", "minimax_m2"):
        return glm_dsa.parse_completion(text)
    raise ValueError(f"unknown chat family {family!r}")


def family_from_architecture(arch: str | None) -> str | None:
    """GGUF ``general.architecture`` / HF ``model_type`` -> chat family."""
    a = (arch or "").lower().replace("_", "-")
    if a.startswith("deepseek"):
        return "deepseek_v4"
    if a.startswith("glm"):
        return "glm_dsa"
    if a.startswith("minimax"):
        return "minimax_m2"
    return None
