"""Convert a LiteLLM ``Choices`` object (or its dict form) into an OpenAI ``Choice``, keeping
tool calls and token log-probs (parity: reference ``src/art/utils/litellm.py``)."""
from __future__ import annotations

from typing import Any

from openai.types.chat.chat_completion import Choice, ChoiceLogprobs
from openai.types.chat.chat_completion_message import ChatCompletionMessage
from openai.types.chat.chat_completion_message_tool_call import ChatCompletionMessageToolCall, Function
from openai.types.chat.chat_completion_token_logprob import ChatCompletionTokenLogprob


def _get(obj: Any, key: str, default=None):
    return obj.get(key, default) if isinstance(obj, dict) else getattr(obj, key, default)


def convert_litellm_choice_to_openai(litellm_choice: Any) -> Choice:
    msg = _get(litellm_choice, "message")
    calls = None
    if _get(msg, "tool_calls"):
        calls = [ChatCompletionMessageToolCall(id=_get(tc, "id") or "", type="function",
                                               function=Function(name=_get(_get(tc, "function"), "name") or "",
                                                                 arguments=_get(_get(tc, "function"), "arguments") or ""))
                 for tc in _get(msg, "tool_calls")]
    message = ChatCompletionMessage(role="assistant", content=_get(msg, "content"), tool_calls=calls)
    lp = _get(litellm_choice, "logprobs")
    logprobs = None
    if lp is not None and _get(lp, "content"):
        logprobs = ChoiceLogprobs(content=[
            ChatCompletionTokenLogprob(token=_get(t, "token"), logprob=_get(t, "logprob"), bytes=_get(t, "bytes"),
                                       top_logprobs=[]) for t in _get(lp, "content")])
    return Choice(index=_get(litellm_choice, "index", 0) or 0, finish_reason=_get(litellm_choice, "finish_reason") or "stop",
                  message=message, logprobs=logprobs)
