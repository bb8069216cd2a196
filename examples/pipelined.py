"""Pipelined rollouts and training with a validation split (the scenarios of the reference's
``dev/swebench/train.ipynb`` and ``examples/temporal_clue/temporal-clue.py``): ``trajectory_group_batches`` keeps later
groups rolling out while the current batch trains; a validation set is gathered concurrently with the first training
batch and logged with ``model.log``; rollouts are re-scored offline, so training runs without the sampled log-probs
(``allow_training_without_logprobs``).

The task is a toy: answer a two-digit sum; the reward is 1 for the right number, else closeness in [0, 0.5).

    python examples/pipelined.py --base-model /models/Qwen2.5-3B-Instruct --steps 10 --groups 4 --group-size 8
"""
from __future__ import annotations

import argparse
import asyncio
import random
import re

import art_b200 as art
from art_b200.local import LocalBackend

from examples.common import add_model_flags, make_model, shutdown


def make_task(rng: random.Random) -> tuple[str, int]:
    a, b = rng.randint(10, 99), rng.randint(10, 99)
    return f"What is {a} + {b}? Answer with the number only.", a + b


def reward_for(text: str | None, answer: int) -> float:
    m = re.search(r"-?\d+", text or "")
    if not m:
        return 0.0
    got = int(m.group())
    return 1.0 if got == answer else max(0.0, 0.5 - abs(got - answer) / 200)


async def rollout(model: art.Model, client, task: tuple[str, int], keep_logprobs: bool) -> art.Trajectory:
    question, answer = task
    messages = [{"role": "user", "content": question}]
    completion = await client.chat.completions.create(model=model.get_inference_name(), messages=messages, max_tokens=8)
    choice = completion.choices[0]
    if not keep_logprobs:
        choice.logprobs = None          # as when rollouts come from an agent framework that drops them
    t = art.Trajectory(messages_and_choices=[*messages, choice], reward=reward_for(choice.message.content, answer))
    t.metrics["correct"] = float(t.reward == 1.0)
    return t.finish()


async def main(a) -> list[float]:
    backend = LocalBackend(in_process=True, path=a.path)
    model = make_model(a)
    rng = random.Random(a.seed)
    history: list[float] = []
    try:
        await model.register(backend)
        client = model.openai_client()
        try:
            start = await model.get_step()
            train_tasks = [make_task(rng) for _ in range(a.groups * max(0, a.steps - start))]
            val_tasks = [make_task(rng) for _ in range(a.val_size)]
            # validation rollouts run while the first training batch is being gathered
            val = asyncio.ensure_future(art.gather_trajectory_groups(
                (art.TrajectoryGroup([rollout(model, client, t, True)]) for t in val_tasks), pbar_desc=None))
            batches = art.trajectory_group_batches(
                (art.TrajectoryGroup(rollout(model, client, t, a.keep_logprobs) for _ in range(a.group_size)) for t in train_tasks),
                batch_size=a.groups, max_concurrent_batches=2, max_batch_exceptions=a.groups // 2, pbar_desc=None)
            async for batch in batches:
                if val is not None:
                    await model.log(await val, split="val")
                    val = None
                rewards = [t.reward for g in batch for t in g.trajectories]
                history.append(sum(rewards) / max(1, len(rewards)))
                print(f"step {await model.get_step()}: mean reward {history[-1]:.3f} over {len(rewards)} rollouts", flush=True)
                await model.train(batch, config=art.TrainConfig(learning_rate=a.lr),
                                  _config={"allow_training_without_logprobs": not a.keep_logprobs})
        finally:
            await client.close()
        return history
    finally:
        await shutdown(backend)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    add_model_flags(ap, "pipelined")
    ap.add_argument("--val-size", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--keep-logprobs", action="store_true", help="train on the sampled log-probs instead of re-scoring")
    ap.set_defaults(lr=5e-5, groups=4, group_size=8, steps=10)
    asyncio.run(main(ap.parse_args()))
