"""2048 (the scenario of the reference's ``examples/2048``): the agent sees the board, answers with a direction, and a
game ends when a tile reaches the goal (reward 2), no move is possible, or the answer is not a direction (reward -1).
Losing games are paid between 0 and 1 by the logarithm of the largest tile and of the board sum, so longer, better
games rank higher inside a group.

    python examples/game_2048.py --base-model /models/Qwen2.5-7B-Instruct --steps 100 --group-size 48
"""
from __future__ import annotations

import argparse
import asyncio
import math
import random
import re

import art_b200 as art
from art_b200.local import LocalBackend

from examples.common import add_model_flags, make_model, shutdown, train_loop

GOAL = 128
SYSTEM = ("You are playing 2048 on a 4x4 board. Each turn answer with exactly one of: left, right, up, down. "
          f"Tiles of equal value merge when they collide; reach {GOAL} to win.")
MOVE_RE = re.compile(r"\b(left|right|up|down)\b", re.I)


def new_board(rng) -> list[list[int]]:
    b = [[0] * 4 for _ in range(4)]
    spawn(b, rng)
    spawn(b, rng)
    return b


def spawn(b, rng) -> None:
    empty = [(r, c) for r in range(4) for c in range(4) if b[r][c] == 0]
    if empty:
        r, c = rng.choice(empty)
        b[r][c] = 2 if rng.random() < 0.9 else 4


def slide_row_left(row: list[int]) -> list[int]:
    tiles = [v for v in row if v]
    out, i = [], 0
    while i < len(tiles):
        if i + 1 < len(tiles) and tiles[i] == tiles[i + 1]:
            out.append(tiles[i] * 2)
            i += 2
        else:
            out.append(tiles[i])
            i += 1
    return out + [0] * (4 - len(out))


def apply_move(b: list[list[int]], direction: str) -> list[list[int]]:
    if direction in ("up", "down"):
        b = [list(col) for col in zip(*b)]
    if direction in ("right", "down"):
        b = [row[::-1] for row in b]
    b = [slide_row_left(row) for row in b]
    if direction in ("right", "down"):
        b = [row[::-1] for row in b]
    if direction in ("up", "down"):
        b = [list(col) for col in zip(*b)]
    return b


def can_move(b) -> bool:
    return any(apply_move(b, d) != b for d in ("left", "right", "up", "down"))


def render(b) -> str:
    return "\n".join("|".join(f"{v or '_':>4}" for v in row) for row in b)


def score(b) -> float:
    top = max(max(r) for r in b)
    if top >= GOAL:
        return 2.0
    total = sum(sum(r) for r in b)
    return 0.8 * (math.log2(top) - 1) / (math.log2(GOAL) - 1) + 0.2 * min(1.0, math.log2(total) / math.log2(16 * GOAL))


async def rollout(model: art.TrainableModel, client, step: int, rng: random.Random | None = None,
                  max_turns: int = 200) -> art.Trajectory:
    rng = rng or random
    b = new_board(rng)
    traj = art.Trajectory(messages_and_choices=[{"role": "system", "content": SYSTEM}], reward=0.0)
    turns = 0
    while turns < max_turns:
        traj.messages_and_choices.append({"role": "user", "content": render(b)})
        completion = await client.chat.completions.create(model=model.get_inference_name(), messages=traj.messages(),
                                                          max_tokens=8)
        choice = completion.choices[0]
        traj.messages_and_choices.append(choice)
        m = MOVE_RE.search(choice.message.content or "")
        if not m:
            traj.reward, traj.metrics["invalid_move"] = -1.0, 1.0
            break
        nb = apply_move(b, m.group(1).lower())
        turns += 1
        if nb != b:
            b = nb
            spawn(b, rng)
        traj.reward = score(b)
        if traj.reward >= 2.0 or not can_move(b):
            break
    traj.metrics["max_tile"] = float(max(max(r) for r in b))
    traj.metrics["turns"] = float(turns)
    traj.metrics["win"] = float(traj.reward >= 2.0)
    return traj.finish()


async def main(a) -> list[float]:
    backend = LocalBackend(in_process=True, path=a.path)
    try:
        return await train_loop(make_model(a), backend, rollout, steps=a.steps, groups=a.groups, group_size=a.group_size,
                                learning_rate=a.lr, keep_best_by="val/reward", max_exceptions=10)
    finally:
        await shutdown(backend)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    add_model_flags(ap, "2048")
    ap.set_defaults(lr=3e-5, group_size=48, steps=100)
    asyncio.run(main(ap.parse_args()))
