"""Public client API: Trajectory / TrajectoryGroup / gather / batches / openai stream folding."""
import asyncio

import pytest
from openai.types.chat.chat_completion import Choice, ChoiceLogprobs
from openai.types.chat.chat_completion_message import ChatCompletionMessage
from openai.types.chat.chat_completion_token_logprob import ChatCompletionTokenLogprob

import art_b200 as art
from art_b200.gather import GatherContext


def make_choice(ids=(5, 6, 7), content="abc"):
    lp = [ChatCompletionTokenLogprob(token=f"token_id:{i}", logprob=-0.5, bytes=None, top_logprobs=[]) for i in ids]
    return Choice(finish_reason="stop", index=0, logprobs=ChoiceLogprobs(content=lp),
                  message=ChatCompletionMessage(role="assistant", content=content))


def traj(reward=1.0, **kw):
    return art.Trajectory(messages_and_choices=[{"role": "user", "content": "hi"}, make_choice()], reward=reward, **kw)


def test_trajectory_messages_and_logging():
    t = traj()
    msgs = t.messages()
    assert msgs[1] == {"role": "assistant", "content": "abc"}
    log = t.for_logging()
    assert [m["trainable"] for m in log["messages"]] == [False, True]
    t.finish()
    assert t.metrics["duration"] >= 0


def test_track_duration_accumulates():
    t = traj()

    async def run():
        async with t.track_duration("llm"):
            await asyncio.sleep(0.01)
        async with t.track_duration("llm"):
            await asyncio.sleep(0.01)

    asyncio.run(run())
    assert t.metrics["llm_duration"] >= 0.02


def test_group_sync_construction_and_exceptions():
    g = art.TrajectoryGroup([traj(1.0), ValueError("boom"), traj(0.0)], metadata={"k": 1})
    assert len(g) == 2 and len(g.exceptions) == 1 and "ValueError" in g.exceptions[0].type
    assert [t.reward for t in g] == [1.0, 0.0]
    again = art.TrajectoryGroup.model_validate(g.model_dump())
    assert len(again) == 2 and again.metadata == {"k": 1}


def test_group_awaitable_and_gather_budget():
    async def rollout(i):
        await asyncio.sleep(0)
        if i == 1:
            raise RuntimeError("bad rollout")
        return traj(float(i))

    async def main(max_exc):
        return await art.gather_trajectory_groups(
            (art.TrajectoryGroup(rollout(i) for i in range(3)) for _ in range(2)), pbar_desc=None, max_exceptions=max_exc)

    groups = asyncio.run(main(2))
    assert [len(g) for g in groups] == [2, 2]
    assert all(len(g.exceptions) == 1 for g in groups)
    assert all("completion_tokens" in t.metrics for g in groups for t in g)
    with pytest.raises(RuntimeError):
        asyncio.run(main(0))


def test_gather_trajectories_returns_exceptions_within_budget():
    async def ok():
        return traj()

    async def bad():
        raise KeyError("x")

    res = asyncio.run(art.gather_trajectories([ok(), bad()], pbar_desc=None, max_exceptions=1))
    assert isinstance(res[0], art.Trajectory) and isinstance(res[1], KeyError)


def test_fractional_exception_budget():
    class Bar:
        total = 10

        def update(self, n): ...
        def set_postfix(self, d): ...

    ctx = GatherContext(pbar=Bar(), max_exceptions=0.25)
    ctx.metric_sums["exceptions"] = 2
    assert not ctx.too_many_exceptions()
    ctx.metric_sums["exceptions"] = 3
    assert ctx.too_many_exceptions()


def test_trajectory_group_batches_pipelines():
    async def group(i):
        await asyncio.sleep(0.001 * (5 - i))
        return art.TrajectoryGroup([traj(float(i))])

    async def main():
        out = []
        async for batch in art.trajectory_group_batches((group(i) for i in range(5)), batch_size=2, pbar_desc=None):
            out.append(len(batch))
        return out

    assert asyncio.run(main()) == [2, 2, 1]


def test_consume_stream_rebuilds_completion():
    from openai.types.chat.chat_completion_chunk import (ChatCompletionChunk, Choice as CChoice, ChoiceDelta,
                                                         ChoiceDeltaToolCall, ChoiceDeltaToolCallFunction)
    from openai.types.completion_usage import CompletionUsage

    from art_b200.openai import consume_chat_completion_stream

    def chunk(delta, finish=None, usage=None, choices=True):
        cs = [CChoice(index=0, delta=delta, finish_reason=finish)] if choices else []
        return ChatCompletionChunk(id="c", created=1, model="m", object="chat.completion.chunk", choices=cs, usage=usage)

    chunks = [
        chunk(ChoiceDelta(role="assistant", content="Hel")),
        chunk(ChoiceDelta(content="lo")),
        chunk(ChoiceDelta(tool_calls=[ChoiceDeltaToolCall(index=0, id="t1", type="function",
                                                           function=ChoiceDeltaToolCallFunction(name="f", arguments='{"a"'))])),
        chunk(ChoiceDelta(tool_calls=[ChoiceDeltaToolCall(index=0, function=ChoiceDeltaToolCallFunction(arguments=": 1}"))]),
              finish="tool_calls"),
        chunk(ChoiceDelta(), choices=False, usage=CompletionUsage(prompt_tokens=3, completion_tokens=2, total_tokens=5)),
    ]

    class Stream:
        def __aiter__(self):
            async def gen():
                for c in chunks:
                    yield c
            return gen()

    comp = asyncio.run(consume_chat_completion_stream(Stream()))
    assert comp.choices[0].message.content == "Hello"
    assert comp.choices[0].message.tool_calls[0].function.arguments == '{"a": 1}'
    assert comp.choices[0].finish_reason == "tool_calls"
    assert comp.usage.prompt_tokens == 3


def test_guided_completion_params():
    from openai.types.chat.chat_completion import ChatCompletion

    from art_b200.guided_completion import get_guided_completion_params

    comp = ChatCompletion(id="x", created=0, model="m", object="chat.completion", choices=[make_choice(content="yes")])
    assert get_guided_completion_params(comp) == (["yes"], None, None)
    tool = {"type": "function", "function": {"name": "move", "parameters": {"type": "object", "properties": {}}}}
    from openai.types.chat.chat_completion_message_tool_call import ChatCompletionMessageToolCall, Function

    ch = make_choice()
    ch.message.tool_calls = [ChatCompletionMessageToolCall(id="1", type="function", function=Function(name="move", arguments='{"x": 2}'))]
    comp = ChatCompletion(id="x", created=0, model="m", object="chat.completion", choices=[ch])
    gc, choice, params = get_guided_completion_params(comp, [tool])
    assert gc is None and choice["function"]["name"] == "move"
    assert params[0]["function"]["parameters"]["properties"]["x"]["const"] == 2 or \
        params[0]["function"]["parameters"]["properties"]["x"].get("enum") == [2]
