"""Smallest loop that shows a learning signal: reward the policy for sampling tokens from a "liked" half of the
vocabulary and watch the mean reward rise over a few GRPO steps.

It is the stand-in for the reference's ``dev/yes-no-maybe.ipynb`` (cell 2) when no pretrained weights are available:
a randomly initialised model cannot answer "maybe", but it can be taught which token ids pay.  The loop is the same
one every ART program runs: register -> rollouts through the OpenAI-compatible server -> ``model.train``.

    python examples/token_preference.py --steps 6            # tiny random model, CPU or GPU
"""
from __future__ import annotations

import argparse
import asyncio
import re
import tempfile

import art_b200 as art
from art_b200.local import LocalBackend

TINY = dict(name="tiny", vocab_size=1024, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
            intermediate_size=384)


def reward_of(choice, liked_below: int) -> float:
    """Share of sampled tokens whose id is liked (token ids come back as ``token_id:N``, as the server is configured
    to return them, reference ``src/art/dev/openai_server.py:20``)."""
    ids = [int(re.sub(r"\D", "", t.token)) for t in choice.logprobs.content]
    return sum(i < liked_below for i in ids) / max(1, len(ids))


async def rollout(model: art.TrainableModel, client, prompt: str, max_tokens: int, liked_below: int) -> art.Trajectory:
    messages = [{"role": "user", "content": prompt}]
    resp = await client.chat.completions.create(model=model.get_inference_name(), messages=messages,
                                                max_tokens=max_tokens, temperature=1.0)
    choice = resp.choices[0]
    return art.Trajectory(messages_and_choices=[*messages, choice], reward=reward_of(choice, liked_below))


async def run(steps: int = 6, groups: int = 8, group_size: int = 8, max_tokens: int = 16, learning_rate: float = 2e-2,
              path: str | None = None, base_model: str = "random:tiny", architecture: dict | None = TINY,
              verbose: bool = True, in_process: bool = True, stop_above: float | None = None) -> list[float]:
    """Returns the mean reward of the rollouts gathered before each training step (plus a final evaluation).

    ``stop_above``: stop early once the mean reward exceeds it (the step at which the reward takes off depends on
    the sampling seeds).  Liked tokens are the ids below 1/16 of the vocabulary: rare enough to need learning, common enough to be found
    by sampling."""
    liked_below = (architecture or TINY)["vocab_size"] // 16
    backend = LocalBackend(in_process=in_process, path=path or tempfile.mkdtemp(prefix="art-token-pref-"))
    # init_std 0.1 instead of 0.02: with the frozen LM head of a random model that small, no adapter could move the
    # next-token distribution far from uniform
    init_args = {"max_seq_length": 2048, "init_std": 0.1}
    if architecture is not None:
        init_args["architecture"] = architecture
    model = art.TrainableModel(name="pref-001", project="token-preference", base_model=base_model,
                               _internal_config={"init_args": init_args,
                                                 "engine_args": {"num_scheduler_steps": 4, "max_model_len": 512}})
    history: list[float] = []
    try:
        await model.register(backend)
        client = model.openai_client()
        prompts = [f"say something nice #{i}" for i in range(groups)]
        for step in range(steps + 1):
            train_groups = await art.gather_trajectory_groups(
                (art.TrajectoryGroup(rollout(model, client, p, max_tokens, liked_below) for _ in range(group_size))
                 for p in prompts), pbar_desc="gather")
            rewards = [t.reward for g in train_groups for t in g.trajectories]
            history.append(sum(rewards) / len(rewards))
            if verbose:
                print(f"step {step}: mean reward {history[-1]:.3f}", flush=True)
            if step == steps or (stop_above is not None and history[-1] > stop_above):
                break
            await model.train(train_groups, config=art.TrainConfig(learning_rate=learning_rate))
        await client.close()
    finally:
        for s in backend._services.values():
            await s.shutdown()
        backend.close()
    return history


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--groups", type=int, default=8)
    ap.add_argument("--group-size", type=int, default=8)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--lr", type=float, default=2e-2)
    a = ap.parse_args()
    hist = asyncio.run(run(a.steps, a.groups, a.group_size, a.max_tokens, a.lr))
    print("mean reward per step:", [round(h, 3) for h in hist])
