"""Rock-paper-scissors through a tool call, against the BASE model (the scenario of the reference's
``examples/rock-paper-tool-use.ipynb``): the trainable model must answer by calling the tool ``play(move)``; its
opponent is the same base model without the adapter, served by the same endpoint under the base model's name, so both
the LoRA and the base model are in use at once.

    python examples/tool_use.py --base-model /models/Qwen2.5-3B-Instruct --steps 20 --group-size 16
"""
from __future__ import annotations

import argparse
import asyncio
import json

import art_b200 as art
from art_b200.local import LocalBackend

from examples.common import add_model_flags, make_model, shutdown, train_loop

MOVES = ("rock", "paper", "scissors")
BEATS = {"rock": "scissors", "paper": "rock", "scissors": "paper"}
TOOLS = [{"type": "function", "function": {
    "name": "play", "description": "Play one move of rock-paper-scissors.",
    "parameters": {"type": "object", "properties": {"move": {"type": "string", "enum": list(MOVES)}}, "required": ["move"]}}}]
PROMPT = "We play rock-paper-scissors. Call the tool `play` with your move."


def move_from(message) -> str | None:
    """The move of a reply: from its tool call if there is one, else the first move named in its text."""
    for call in getattr(message, "tool_calls", None) or []:
        try:
            m = json.loads(call.function.arguments).get("move")
        except (json.JSONDecodeError, AttributeError):
            continue
        if m in MOVES:
            return m
    text = (getattr(message, "content", None) or "").lower()
    found = [(text.find(m), m) for m in MOVES if m in text]
    return min(found)[1] if found else None


def outcome(mine: str | None, theirs: str | None) -> float:
    if mine is None:
        return -1.0
    if theirs is None or BEATS[mine] == theirs:
        return 1.0
    return 0.5 if mine == theirs else 0.0


async def rollout(model: art.TrainableModel, client, step: int) -> art.Trajectory:
    messages = [{"role": "user", "content": PROMPT}]
    mine = await client.chat.completions.create(model=model.get_inference_name(), messages=messages, tools=TOOLS,
                                                max_tokens=48)
    # the opponent: the base model, same server, no adapter
    theirs = await client.chat.completions.create(model=model.base_model, messages=messages, tools=TOOLS, max_tokens=48)
    traj = art.Trajectory(messages_and_choices=[*messages, mine.choices[0]], tools=TOOLS, reward=0.0)
    m, o = move_from(mine.choices[0].message), move_from(theirs.choices[0].message)
    traj.reward = outcome(m, o)
    traj.metrics["used_tool"] = float(bool(mine.choices[0].message.tool_calls))
    traj.metrics["opponent_moved"] = float(o is not None)
    return traj.finish()


async def main(a) -> list[float]:
    backend = LocalBackend(in_process=True, path=a.path)
    try:
        return await train_loop(make_model(a), backend, rollout, steps=a.steps, groups=a.groups, group_size=a.group_size,
                                learning_rate=a.lr, max_exceptions=a.group_size // 4)
    finally:
        await shutdown(backend)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    add_model_flags(ap, "rock-paper-tool-use")
    ap.set_defaults(lr=5e-5, group_size=16, steps=20)
    asyncio.run(main(ap.parse_args()))
