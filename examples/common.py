"""Shared plumbing of the example programs: model construction from command-line flags and the train loop.

Every example defines a ``rollout(model, client, step) -> art.Trajectory`` coroutine; :func:`train_loop` is the loop
all of the reference's examples share (``examples/2048/2048.py:46-68``, ``examples/tic_tac_toe/tic-tac-toe.py``):
gather groups of rollouts, optionally keep only the best checkpoints, train, repeat until ``steps``.
"""
from __future__ import annotations

import argparse
from typing import Awaitable, Callable

import art_b200 as art
from art_b200.local import LocalBackend

TINY = dict(name="tiny", vocab_size=1024, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
            intermediate_size=384)


def add_model_flags(ap: argparse.ArgumentParser, project: str) -> None:
    ap.add_argument("--base-model", default="random:tiny",
                    help="local Hugging Face directory of the base model, or random:<preset> for random weights")
    ap.add_argument("--name", default="001")
    ap.add_argument("--project", default=project)
    ap.add_argument("--path", default=None, help="where checkpoints and logs go (default: ./.art)")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--groups", type=int, default=1)
    ap.add_argument("--group-size", type=int, default=8)
    ap.add_argument("--lr", type=float, default=3e-5)
    ap.add_argument("--max-seq-length", type=int, default=8192)


def make_model(a) -> art.TrainableModel:
    init_args: dict = {"max_seq_length": a.max_seq_length}
    if a.base_model == "random:tiny":
        init_args["architecture"] = TINY
    return art.TrainableModel(name=a.name, project=a.project, base_model=a.base_model,
                              _internal_config={"init_args": init_args,
                                                "engine_args": {"max_model_len": a.max_seq_length}})


async def train_loop(model: art.TrainableModel, backend: LocalBackend,
                     rollout: Callable[[art.TrainableModel, object, int], Awaitable[art.Trajectory]], *, steps: int,
                     groups: int, group_size: int, learning_rate: float, keep_best_by: str | None = None,
                     max_exceptions: int = 0, verbose: bool = True) -> list[float]:
    """Returns the mean reward of each step's rollouts."""
    await model.register(backend)
    client = model.openai_client()
    history = []
    try:
        for step in range(await model.get_step(), steps):
            train_groups = await art.gather_trajectory_groups(
                (art.TrajectoryGroup(rollout(model, client, step) for _ in range(group_size)) for _ in range(groups)),
                pbar_desc="gather", max_exceptions=max_exceptions)
            rewards = [t.reward for g in train_groups for t in g.trajectories]
            history.append(sum(rewards) / max(1, len(rewards)))
            if verbose:
                print(f"step {step}: mean reward {history[-1]:.3f} over {len(rewards)} rollouts", flush=True)
            if keep_best_by:
                await model.delete_checkpoints(best_checkpoint_metric=keep_best_by)
            await model.train(train_groups, config=art.TrainConfig(learning_rate=learning_rate))
    finally:
        await client.close()
    return history


async def shutdown(backend: LocalBackend) -> None:
    for s in getattr(backend, "_services", {}).values():
        await s.shutdown()
    backend.close()
