"""Run one rollout function many times against a model and average the rewards
(parity: reference ``src/art/utils/benchmark_rollout.py:8-28``)."""
from __future__ import annotations

from typing import Awaitable, Callable

from ..gather import gather_trajectories
from ..trajectories import Trajectory


async def benchmark_rollout(model: str, num_rollouts: int,
                            rollout: Callable[[str, int, bool], Awaitable[Trajectory]]) -> float:
    results = await gather_trajectories([rollout(model, i, False) for i in range(num_rollouts)],
                                        pbar_desc="Benchmarking rollout", max_exceptions=num_rollouts)
    rewards = [t.reward for t in results if isinstance(t, Trajectory)]
    return sum(rewards) / len(rewards) if rewards else 0.0
