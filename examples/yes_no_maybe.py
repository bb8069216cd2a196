"""The reference's smallest training loop (``dev/yes-no-maybe.ipynb`` cell 2): the model is asked to respond with
yes, no or maybe and is paid 0.5 / 0.75 / 1.0 for exactly those answers, nothing otherwise; it learns to say "maybe".

    python examples/yes_no_maybe.py --base-model /models/Qwen2.5-7B-Instruct --steps 20
"""
from __future__ import annotations

import argparse
import asyncio

import art_b200 as art
from art_b200.local import LocalBackend

from examples.common import add_model_flags, make_model, shutdown, train_loop

REWARDS = {"yes": 0.5, "no": 0.75, "maybe": 1.0}


def prompts() -> list[str]:
    out = []
    word_lists = [["yes", "no", "maybe"], ["maybe", "yes", "no"], ["no", "yes", "maybe"], ["yes", "maybe", "no"],
                  ["yes", "no"], ["maybe", "no"], ["no", "maybe"], ["no", "yes"], ["yes", "no"]]
    for prefix in ("respond", "just respond"):
        for quoted in (True, False):
            for words in word_lists:
                shown = [f"'{w}'" if quoted else w for w in words]
                tail = ", ".join(shown) if len(words) == 3 else " or ".join(words)
                out.append(f"{prefix} with {tail}")
    return out


def reward_for(content: str | None) -> float:
    return REWARDS.get((content or "").strip(), 0.0)


def make_rollout(prompt_list: list[str], no_thinking: bool = False):
    # new "thinking" model families (the reference's dev/new_models/qwen3_try.py): switch the reasoning preamble off
    # through the chat template, so that the answer is the one word the reward looks for
    extra = {"extra_body": {"chat_template_kwargs": {"enable_thinking": False}}} if no_thinking else {}

    async def rollout(model: art.TrainableModel, client, step: int) -> art.Trajectory:
        rollout.calls += 1
        prompt = prompt_list[(rollout.calls // rollout.group_size) % len(prompt_list)]
        messages: art.Messages = [{"role": "user", "content": prompt}]
        completion = await client.chat.completions.create(messages=messages, model=model.get_inference_name(),
                                                          max_tokens=100, timeout=100, **extra)
        choice = completion.choices[0]
        return art.Trajectory(messages_and_choices=[*messages, choice], reward=reward_for(choice.message.content))

    rollout.calls, rollout.group_size = -1, 1
    return rollout


async def main(a) -> list[float]:
    backend = LocalBackend(in_process=True, path=a.path)
    rollout = make_rollout(prompts(), getattr(a, "no_thinking", False))
    rollout.group_size = a.group_size
    try:
        return await train_loop(make_model(a), backend, rollout, steps=a.steps, groups=a.groups, group_size=a.group_size,
                                learning_rate=a.lr)
    finally:
        await shutdown(backend)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    add_model_flags(ap, "yes-no-maybe")
    ap.add_argument("--no-thinking", action="store_true",
                    help="pass chat_template_kwargs={'enable_thinking': False} (Qwen3-style chat templates)")
    ap.set_defaults(lr=1e-4, groups=36, group_size=32, steps=1000)
    asyncio.run(main(ap.parse_args()))
