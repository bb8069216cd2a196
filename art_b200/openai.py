"""AsyncOpenAI client instrumentation (parity: reference ``src/art/openai.py:19-172``).

Inside a ``gather_*`` call that wants live completion-token totals, every
``chat.completions.create`` is switched to streaming with usage reporting; the stream is
folded back into an ordinary ``ChatCompletion`` so rollout code does not notice.
"""
from __future__ import annotations

from typing import Any, AsyncIterator, Callable

import openai
from openai.types.chat.chat_completion import ChatCompletion, Choice, ChoiceLogprobs
from openai.types.chat.chat_completion_chunk import ChatCompletionChunk
from openai.types.chat.chat_completion_message import ChatCompletionMessage, FunctionCall
from openai.types.chat.chat_completion_message_tool_call import ChatCompletionMessageToolCall, Function

from .gather import get_gather_context


def _count_logprob_tokens(chunk: ChatCompletionChunk) -> int:
    n = 0
    for c in chunk.choices:
        if c.logprobs:
            n += len(c.logprobs.content or c.logprobs.refusal or [])
    return n


def _report_usage(completion: ChatCompletion) -> None:
    ctx = get_gather_context()
    if completion.usage is not None:
        ctx.metric_sums["prompt_tokens"] += completion.usage.prompt_tokens
        ctx.metric_divisors["prompt_tokens"] += 1


def patch_openai(client: openai.AsyncOpenAI) -> openai.AsyncOpenAI:
    original = client.chat.completions.create

    async def create(*args: Any, **kwargs: Any):
        caller_wants_stream = bool(kwargs.get("stream", False))
        ctx = get_gather_context()
        if ctx.pbar_total_completion_tokens:
            kwargs["stream"] = True
            kwargs["stream_options"] = {"include_usage": True}
        result = await original(*args, **kwargs)
        if not isinstance(result, AsyncIterator):
            _report_usage(result)
            return result
        if caller_wants_stream:
            return result

        def on_chunk(chunk: ChatCompletionChunk, _partial: ChatCompletion) -> None:
            c = get_gather_context()
            if c.pbar_total_completion_tokens:
                c.metric_sums["total_completion_tokens"] += _count_logprob_tokens(chunk)
                c.update_pbar(n=0)

        completion = await consume_chat_completion_stream(result, on_chunk)
        _report_usage(completion)
        return completion

    client.chat.completions.create = create  # type: ignore[method-assign]
    return client


def _merge_choice(dst: Choice, src) -> None:
    dst.finish_reason = src.finish_reason or "stop"
    if src.logprobs:
        if dst.logprobs is None:
            dst.logprobs = ChoiceLogprobs()
        for attr in ("content", "refusal"):
            extra = getattr(src.logprobs, attr)
            if extra:
                cur = getattr(dst.logprobs, attr)
                if cur is None:
                    setattr(dst.logprobs, attr, list(extra))
                else:
                    cur.extend(extra)
    d = src.delta
    if d.content:
        dst.message.content = (dst.message.content or "") + d.content
    if d.refusal:
        dst.message.refusal = (dst.message.refusal or "") + d.refusal
    if d.function_call:
        if dst.message.function_call is None:
            dst.message.function_call = FunctionCall(arguments="", name="")
        dst.message.function_call.name += d.function_call.name or ""
        dst.message.function_call.arguments += d.function_call.arguments or ""
    if d.tool_calls:
        if dst.message.tool_calls is None:
            dst.message.tool_calls = []
        calls = dst.message.tool_calls
        for tc in d.tool_calls:
            while len(calls) <= tc.index:
                calls.append(ChatCompletionMessageToolCall(id="", function=Function(arguments="", name=""), type="function"))
            if tc.id:
                calls[tc.index].id = tc.id
            if tc.function:
                if tc.function.name:
                    calls[tc.index].function.name = tc.function.name
                if tc.function.arguments:
                    calls[tc.index].function.arguments += tc.function.arguments
    reasoning = getattr(d, "reasoning", None)
    if reasoning:
        setattr(dst.message, "reasoning", (getattr(dst.message, "reasoning", "") or "") + reasoning)


async def consume_chat_completion_stream(
    stream, on_chunk: Callable[[ChatCompletionChunk, ChatCompletion], Any] | None = None
) -> ChatCompletion:
    """Fold a stream of chunks into the ``ChatCompletion`` a non-streaming call would return.

    ``on_chunk`` may raise ``StopIteration`` to end consumption early.
    """
    completion: ChatCompletion | None = None
    async for chunk in stream:
        if completion is None:
            completion = ChatCompletion(
                id=chunk.id, created=chunk.created, model=chunk.model, object="chat.completion",
                choices=[Choice(finish_reason="stop", index=c.index,
                                logprobs=ChoiceLogprobs() if c.logprobs else None,
                                message=ChatCompletionMessage(role="assistant")) for c in chunk.choices],
            )
        by_index = {c.index: c for c in completion.choices}
        for src in chunk.choices:
            if src.index not in by_index:
                new = Choice(finish_reason="stop", index=src.index, logprobs=None,
                             message=ChatCompletionMessage(role="assistant"))
                completion.choices.append(new)
                by_index[src.index] = new
            _merge_choice(by_index[src.index], src)
        completion.service_tier = chunk.service_tier
        completion.system_fingerprint = chunk.system_fingerprint
        if chunk.usage is not None or completion.usage is None:
            completion.usage = chunk.usage
        if on_chunk:
            try:
                on_chunk(chunk, completion)
            except StopIteration:
                await stream.close()
                break
    assert completion is not None, "stream produced no chunks"
    return completion
