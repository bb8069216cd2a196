"""Benchmark a trained model against prompted comparison models through the same API (the scenario of the
reference's ``examples/benchmarking_comparison_models.py``): a comparison model is an ``art.Model`` that points at any
OpenAI-compatible endpoint; its validation rollouts are logged with ``model.log`` next to the trained model's, and
the benchmark loaders and charts read both from the same project directory.

Offline, the "comparison model" here is the untrained base model served by the trainable model's own endpoint; with
network access any hosted model works (``--compare-url https://... --compare-key ... --compare-model gpt-4o``).

    python examples/comparison_models.py --base-model /models/Qwen2.5-3B-Instruct --steps 5 --chart progress.svg
"""
from __future__ import annotations

import argparse
import asyncio
import random

import art_b200 as art
from art_b200.local import LocalBackend
from art_b200.utils.benchmarking.charts import percentage_comparison_bar_chart, training_progress_chart
from art_b200.utils.benchmarking.load_trajectories import load_trajectories
from art_b200.utils.benchmarking.types import BenchmarkModelKey

from examples.common import add_model_flags, make_model, shutdown
from examples.pipelined import make_task, reward_for


async def rollout(model: art.Model, task: tuple[str, int]) -> art.Trajectory:
    question, answer = task
    messages = [{"role": "user", "content": question}]
    client = model.openai_client()
    completion = await client.chat.completions.create(model=model.get_inference_name(), messages=messages, max_tokens=8)
    choice = completion.choices[0]
    t = art.Trajectory(messages_and_choices=[*messages, choice], reward=reward_for(choice.message.content, answer))
    t.metrics["correct"] = float(t.reward == 1.0)
    return t.finish()


async def evaluate(model: art.Model, tasks: list[tuple[str, int]]) -> float:
    """Roll the validation tasks out with ``model``, log them under split ``val``, return the mean reward."""
    groups = await art.gather_trajectory_groups((art.TrajectoryGroup([rollout(model, t)]) for t in tasks), pbar_desc=None)
    await model.log(groups, split="val")
    rewards = [t.reward for g in groups for t in g.trajectories]
    return sum(rewards) / max(1, len(rewards))


async def main(a) -> dict:
    backend = LocalBackend(in_process=True, path=a.path)
    model = make_model(a)
    rng = random.Random(a.seed)
    val_tasks = [make_task(rng) for _ in range(a.val_size)]
    scores: dict[str, list[float]] = {model.name: []}
    try:
        await model.register(backend)
        base_url, api_key = model.inference_base_url, model.inference_api_key
        compare = art.Model(name=a.compare_name, project=a.project,
                            inference_model_name=a.compare_model or model.base_model,
                            inference_base_url=a.compare_url or base_url, inference_api_key=a.compare_key or api_key)
        await compare.register(backend)
        scores[compare.name] = [await evaluate(compare, val_tasks)]          # prompted models are evaluated once
        for step in range(await model.get_step(), a.steps):
            scores[model.name].append(await evaluate(model, val_tasks))
            groups = await art.gather_trajectory_groups(
                (art.TrajectoryGroup(rollout(model, make_task(rng)) for _ in range(a.group_size)) for _ in range(a.groups)),
                pbar_desc=None)
            await model.train(groups, config=art.TrainConfig(learning_rate=a.lr))
        scores[model.name].append(await evaluate(model, val_tasks))
        df = await load_trajectories(a.project, art_path=a.path)
        keys = [BenchmarkModelKey(model.name, "Trained", "val"), BenchmarkModelKey(compare.name, "Prompted", "val")]
        if a.chart:
            training_progress_chart(df, "reward", keys, title="Validation reward", path=a.chart)
        if a.bars:
            percentage_comparison_bar_chart(df, "correct", keys, title="Exact answers", path=a.bars)
        return {"scores": scores, "rows": len(df)}
    finally:
        await model.openai_client().close()
        await shutdown(backend)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    add_model_flags(ap, "comparison-models")
    ap.add_argument("--compare-name", default="prompted-baseline")
    ap.add_argument("--compare-model", default=None, help="model name at the comparison endpoint (default: the base model)")
    ap.add_argument("--compare-url", default=None, help="OpenAI-compatible endpoint (default: this run's own server)")
    ap.add_argument("--compare-key", default=None)
    ap.add_argument("--val-size", type=int, default=16)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--chart", default=None, help="write the training-progress chart (SVG) here")
    ap.add_argument("--bars", default=None, help="write the comparison bar chart (SVG) here")
    ap.set_defaults(lr=5e-5, groups=2, group_size=8, steps=5)
    print(asyncio.run(main(ap.parse_args())))
