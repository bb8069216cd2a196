"""Per-step statistics over trajectory groups (parity: reference
``src/art/utils/old_benchmarking/calculate_step_metrics.py:5-21``)."""
from __future__ import annotations

import math


def calculate_step_std_dev(trajectory_groups) -> float:
    """Mean over groups of the population standard deviation of the rewards inside a group; groups with fewer than
    two scored trajectories do not count.  This is the learning-signal gauge logged as ``reward_std_dev``: GRPO
    has no gradient for a group whose rewards are all equal."""
    stds = []
    for group in trajectory_groups:
        rewards = [t.reward for t in group.trajectories if not isinstance(t, BaseException)]
        if len(rewards) > 1:
            mean = sum(rewards) / len(rewards)
            stds.append(math.sqrt(sum((r - mean) ** 2 for r in rewards) / len(rewards)))
    return sum(stds) / len(stds) if stds else 0.0
