"""Trajectory groups -> token-level training records (parity: reference
``src/art/local/tokenize.py:11-196``).

Per group: population mean/std of rewards -> advantage ``(r - mean) / (std + 1e-6)``;
zero-advantage trajectories are dropped; the longest common token prefix of the group's
records is the shared prompt.  Per trajectory: the conversation is rendered once with a
sentinel token in place of every sampled ``Choice`` and the sampled token ids (parsed from
``token_id:N`` strings) with their log-probs are spliced in, so training sees the exact
sampled ids rather than a re-tokenisation.

Differences from the reference, on purpose: randomness (prompt ids, shuffle) comes from an
explicit ``random.Random`` so packing is reproducible, and when training without
log-probs the template's assistant-token mask is used if the tokenizer provides one.
"""
from __future__ import annotations

import math
import random
from collections.abc import Mapping
from dataclasses import dataclass, replace
from typing import Any, Iterator

from openai.types.chat.chat_completion import Choice

from ..trajectories import Trajectory, TrajectoryGroup

_INT64_MIN, _INT64_MAX = -(2 ** 63), 2 ** 63 - 1


@dataclass
class TokenizedResult:
    trajectory: Trajectory
    advantage: float
    chat: str
    tokens: list[str]
    token_ids: list[int]
    input_pos: list[int]
    assistant_mask: list[int]
    logprobs: list[float]
    prompt_id: int = 0
    prompt_length: int = 0

    def without_prompt(self) -> "TokenizedResult":
        n = self.prompt_length
        return replace(self, tokens=self.tokens[n:], token_ids=self.token_ids[n:], input_pos=self.input_pos[n:],
                       assistant_mask=self.assistant_mask[n:], logprobs=self.logprobs[n:], prompt_length=0)


def group_advantages(rewards: list[float]) -> list[float]:
    """GRPO advantages with the population standard deviation."""
    n = len(rewards)
    mean = sum(rewards) / n
    std = math.sqrt(sum((r - mean) ** 2 for r in rewards) / n)
    return [(r - mean) / (std + 1e-6) for r in rewards]


def common_prefix_length(seqs: list[list[int]]) -> int:
    if not seqs:
        return 0
    n = 0
    for column in zip(*seqs):
        if any(v != column[0] for v in column):
            break
        n += 1
    return n


def tokenize_trajectory_groups(tokenizer, trajectory_groups: list[TrajectoryGroup],
                               allow_training_without_logprobs: bool,
                               rng: random.Random | None = None) -> Iterator[TokenizedResult]:
    rng = rng or random
    for group in trajectory_groups:
        if not len(group):
            continue
        advantages = group_advantages([t.reward for t in group])
        results: list[TokenizedResult] = []
        for traj, adv in zip(group, advantages):
            if adv == 0:
                continue
            r = tokenize_trajectory(tokenizer, traj, adv, allow_training_without_logprobs)
            if r is not None:
                results.append(r)
        prompt_id = rng.randint(_INT64_MIN, _INT64_MAX)
        prompt_length = common_prefix_length([r.token_ids for r in results])
        for r in results:
            r.prompt_id = prompt_id
            r.prompt_length = prompt_length
        rng.shuffle(results)
        yield from results


def _last_trainable_index(items: list[Any], allow_without_logprobs: bool) -> int:
    last = -1
    for i, m in enumerate(items):
        if isinstance(m, dict):
            if allow_without_logprobs and m.get("role") == "assistant":
                last = i
        elif m.logprobs or allow_without_logprobs:
            last = i
    return last


def tokenize_trajectory(tokenizer, trajectory: Trajectory, advantage: float,
                        allow_training_without_logprobs: bool) -> TokenizedResult | None:
    last = _last_trainable_index(trajectory.messages_and_choices, allow_training_without_logprobs)
    if last < 0:
        return None
    trajectory = trajectory.model_copy(update={"messages_and_choices": trajectory.messages_and_choices[: last + 1]})
    messages = trajectory.messages()
    tools = trajectory.tools
    chat = tokenizer.apply_chat_template(messages, tools=tools, tokenize=False)
    original_ids = tokenizer.apply_chat_template(messages, tools=tools)
    if isinstance(original_ids, Mapping):      # newer tokenizer libraries return the dictionary form by default
        original_ids = original_ids["input_ids"]
    used = set(original_ids)
    sentinel_id = next(i for i in range(int(tokenizer.vocab_size) - 1, -1, -1) if i not in used)
    sentinel_text = tokenizer.decode(sentinel_id)
    templated = [m if isinstance(m, dict) else {"role": "assistant", "content": sentinel_text}
                 for m in trajectory.messages_and_choices]
    rendered = tokenizer.apply_chat_template(templated, tools=tools, return_dict=True,
                                             return_assistant_tokens_mask=allow_training_without_logprobs)
    token_ids: list[int] = list(rendered["input_ids"])
    if allow_training_without_logprobs:
        mask = rendered.get("assistant_masks")
        assistant_mask = list(mask) if mask is not None else list(rendered["attention_mask"])
    else:
        assistant_mask = [0] * len(token_ids)
    logprobs = [float("nan")] * len(token_ids)
    for item in trajectory.messages_and_choices:
        if isinstance(item, dict):
            continue
        choice: Choice = item
        if not (choice.logprobs or allow_training_without_logprobs):
            raise AssertionError("Chat completion choices must have logprobs")
        if not choice.logprobs:
            continue
        tlps = choice.logprobs.content or choice.logprobs.refusal or []
        at = token_ids.index(sentinel_id)
        token_ids[at:at + 1] = [int(t.token.split(":")[1]) for t in tlps]
        logprobs[at:at + 1] = [t.logprob for t in tlps]
        assistant_mask[at:at + 1] = [1] * len(tlps)
    return TokenizedResult(
        trajectory=trajectory, advantage=advantage, chat=chat,
        tokens=[tokenizer.decode(i) for i in token_ids], token_ids=token_ids,
        input_pos=list(range(len(token_ids))), assistant_mask=assistant_mask, logprobs=logprobs,
    )
