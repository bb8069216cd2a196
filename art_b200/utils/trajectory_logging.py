"""YAML (de)serialisation of trajectory groups (parity: reference
``src/art/utils/trajectory_logging.py:9-84``).  Token log-probs are dropped on write."""
from __future__ import annotations

from typing import Any

import yaml
from openai.types.chat.chat_completion import Choice

from ..trajectories import Trajectory, TrajectoryGroup


def message_or_choice_to_dict(message_or_choice) -> dict[str, Any]:
    d = dict(message_or_choice) if isinstance(message_or_choice, dict) else message_or_choice.to_dict()
    d.pop("logprobs", None)
    return d


def trajectory_to_dict(trajectory: Trajectory) -> dict[str, Any]:
    return {
        "reward": trajectory.reward,
        "metrics": dict(trajectory.metrics),
        "metadata": dict(trajectory.metadata),
        "messages_and_choices": [message_or_choice_to_dict(m) for m in trajectory.messages_and_choices],
        "logs": list(trajectory.logs),
    }


def trajectory_group_to_dict(trajectory_group: TrajectoryGroup) -> dict[str, Any]:
    return {"trajectories": [trajectory_to_dict(t) for t in trajectory_group.trajectories if isinstance(t, Trajectory)],
            "metadata": dict(trajectory_group.metadata)}


def serialize_trajectory_groups(trajectory_groups: list[TrajectoryGroup]) -> str:
    return yaml.safe_dump([trajectory_group_to_dict(g) for g in trajectory_groups], sort_keys=True)


def dict_to_message_or_choice(d: dict[str, Any]):
    if "message" in d:
        return Choice(**d)
    if d.get("role") not in ("system", "user", "assistant", "tool", "developer", "function"):
        raise ValueError(f"Unknown message role: {d.get('role')}")
    return dict(d)


def dict_to_trajectory(d: dict[str, Any]) -> Trajectory:
    return Trajectory(
        messages_and_choices=[dict_to_message_or_choice(m) for m in d["messages_and_choices"]],
        reward=d["reward"], metrics=d.get("metrics", {}), metadata=d.get("metadata", {}), logs=d.get("logs", []),
    )


def dict_to_trajectory_group(d: dict[str, Any]) -> TrajectoryGroup:
    return TrajectoryGroup([dict_to_trajectory(t) for t in d["trajectories"]], metadata=d.get("metadata", {}), exceptions=[])


def deserialize_trajectory_groups(serialized: str) -> list[TrajectoryGroup]:
    return [dict_to_trajectory_group(g) for g in (yaml.safe_load(serialized) or [])]
