"""Tic-tac-toe self-play (the scenario of the reference's ``examples/tic_tac_toe_self_play``): the model plays both
sides, so one game yields TWO trajectories (X's view and O's view); the trajectories of all games are grouped by side
(all X trajectories in one group, all O trajectories in another) and a scripted teacher picks a fraction of the moves,
which the student is then forced to reproduce through ``guided_choice`` (its log-probs come back as for sampled moves).

    python examples/self_play.py --base-model /models/Qwen2.5-3B-Instruct --steps 30 --group-size 32 --teacher 0.25
"""
from __future__ import annotations

import argparse
import asyncio
import random

import art_b200 as art
from art_b200.local import LocalBackend

from examples.common import add_model_flags, make_model, shutdown
from examples.tic_tac_toe import LINES, parse_move, render, winner

SYSTEM = ("You are playing tic-tac-toe as {side}. Squares are named by column letter and row number, A1 to C3. "
          "Answer with the name of one empty square and nothing else.")


def teacher_move(board: list[str], side: str) -> str:
    """Win if possible, else block, else centre, else the first free square; as a square name."""
    other = "O" if side == "X" else "X"
    free = [i for i, s in enumerate(board) if s == "."]
    for who in (side, other):
        for a, b, c in LINES:
            line = [board[a], board[b], board[c]]
            if line.count(who) == 2 and line.count(".") == 1:
                idx = (a, b, c)[line.index(".")]
                return "ABC"[idx % 3] + str(idx // 3 + 1)
    idx = 4 if 4 in free else free[0]
    return "ABC"[idx % 3] + str(idx // 3 + 1)


async def play_game(model: art.TrainableModel, client, teacher: float, rng: random.Random) -> list[art.Trajectory]:
    """One game; returns [trajectory of X, trajectory of O]."""
    board = ["."] * 9
    trajs = {s: art.Trajectory(messages_and_choices=[{"role": "system", "content": SYSTEM.format(side=s)}], reward=0.0)
             for s in "XO"}
    side, result = "X", None
    while result is None:
        t = trajs[side]
        t.messages_and_choices.append({"role": "user", "content": render(board)})
        extra = {}
        if rng.random() < teacher:        # the teacher decides; the student's reply is forced to that move
            extra = {"extra_body": {"guided_choice": [teacher_move(board, side)]}}
            t.metrics["guided_moves"] = t.metrics.get("guided_moves", 0.0) + 1.0
        completion = await client.chat.completions.create(model=model.get_inference_name(), messages=t.messages(),
                                                          max_tokens=8, **extra)
        choice = completion.choices[0]
        t.messages_and_choices.append(choice)
        idx = parse_move(choice.message.content, board)
        if idx is None:                    # illegal or unparsable: this side loses at once
            result = "O" if side == "X" else "X"
            t.metrics["illegal_move"] = 1.0
            break
        board[idx] = side
        result = winner(board)
        side = "O" if side == "X" else "X"
    for s, t in trajs.items():
        t.reward = 0.5 if result == "draw" else (1.0 if result == s else 0.0)
        if t.metrics.get("illegal_move"):
            t.reward = -1.0
        t.finish()
    return [trajs["X"], trajs["O"]]


async def main(a) -> list[float]:
    backend = LocalBackend(in_process=True, path=a.path)
    model = make_model(a)
    rng = random.Random(a.seed)
    history = []
    try:
        await model.register(backend)
        client = model.openai_client()
        try:
            for step in range(await model.get_step(), a.steps):
                games = await art.gather_trajectories((play_game(model, client, a.teacher, rng) for _ in range(a.group_size)),
                                                      pbar_desc="games", max_exceptions=a.group_size // 4)
                games = [g for g in games if isinstance(g, list)]
                # groups by index: the X trajectories of all games compete with one another, and so do the O ones
                groups = [art.TrajectoryGroup(g[i] for g in games) for i in range(2)]
                rewards = [t.reward for g in groups for t in g.trajectories]
                history.append(sum(rewards) / max(1, len(rewards)))
                print(f"step {step}: mean reward {history[-1]:.3f} over {len(games)} games", flush=True)
                await model.train(groups, config=art.TrainConfig(learning_rate=a.lr))
        finally:
            await client.close()
        return history
    finally:
        await shutdown(backend)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    add_model_flags(ap, "tic-tac-toe-self-play")
    ap.add_argument("--teacher", type=float, default=0.25, help="share of moves decided by the scripted teacher")
    ap.add_argument("--seed", type=int, default=0)
    ap.set_defaults(lr=5e-5, group_size=32, steps=30)
    asyncio.run(main(ap.parse_args()))
