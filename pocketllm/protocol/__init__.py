from .chat import ChatRequest, extract_tool_calls, split_reasoning, truncate_at_stop
from .prompt import TokenizerHandle, encode_chat_prompt
from .requests import build_chat_request, build_completion_request

__all__ = ["ChatRequest", "TokenizerHandle", "build_chat_request", "build_completion_request", "encode_chat_prompt",
           "extract_tool_calls", "split_reasoning", "truncate_at_stop"]
