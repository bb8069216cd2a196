"""Tic-tac-toe against a random opponent (the scenario of the reference's ``examples/tic_tac_toe``): the agent plays
X, answers each turn with a square like ``B2``, and is paid 1 for a win, 0.5 for a draw, 0 for a loss and -1 for an
illegal or unparsable move (which ends the game), plus a small bonus for surviving longer.

    python examples/tic_tac_toe.py --base-model /models/Qwen2.5-3B-Instruct --steps 50 --group-size 48
"""
from __future__ import annotations

import argparse
import asyncio
import random
import re

import art_b200 as art
from art_b200.local import LocalBackend

from examples.common import add_model_flags, make_model, shutdown, train_loop

LINES = [(0, 1, 2), (3, 4, 5), (6, 7, 8), (0, 3, 6), (1, 4, 7), (2, 5, 8), (0, 4, 8), (2, 4, 6)]
SYSTEM = ("You are playing tic-tac-toe as X. Squares are named by column letter and row number, A1 to C3. "
          "Answer with the name of one empty square and nothing else.")


def render(board: list[str]) -> str:
    rows = ["   A B C"]
    for r in range(3):
        rows.append(f"{r + 1}  " + " ".join(board[r * 3 + c] for c in range(3)))
    return "\n".join(rows)


def winner(board: list[str]) -> str | None:
    for a, b, c in LINES:
        if board[a] != "." and board[a] == board[b] == board[c]:
            return board[a]
    return "draw" if "." not in board else None


def parse_move(text: str | None, board: list[str]) -> int | None:
    m = re.search(r"\b([A-Ca-c])\s*([1-3])\b", text or "")
    if not m:
        return None
    idx = (int(m.group(2)) - 1) * 3 + "ABC".index(m.group(1).upper())
    return idx if board[idx] == "." else None


async def rollout(model: art.TrainableModel, client, step: int, rng: random.Random | None = None) -> art.Trajectory:
    rng = rng or random
    board = ["."] * 9
    traj = art.Trajectory(messages_and_choices=[{"role": "system", "content": SYSTEM}], reward=0.0)
    moves = 0
    while True:
        traj.messages_and_choices.append({"role": "user", "content": render(board)})
        completion = await client.chat.completions.create(model=model.get_inference_name(), messages=traj.messages(),
                                                          max_tokens=8)
        choice = completion.choices[0]
        traj.messages_and_choices.append(choice)
        idx = parse_move(choice.message.content, board)
        if idx is None:
            traj.reward, traj.metrics["illegal_move"] = -1.0 + 0.05 * moves, 1.0
            break
        board[idx] = "X"
        moves += 1
        w = winner(board)
        if w is None:
            board[rng.choice([i for i, s in enumerate(board) if s == "."])] = "O"
            w = winner(board)
        if w is not None:
            traj.reward = {"X": 1.0, "draw": 0.5, "O": 0.0}[w] + 0.02 * moves
            traj.metrics["win"] = float(w == "X")
            break
    traj.metrics["moves"] = float(moves)
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
    add_model_flags(ap, "tic-tac-toe")
    ap.set_defaults(lr=5e-5, group_size=48, steps=50)
    asyncio.run(main(ap.parse_args()))
