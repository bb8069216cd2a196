"""YAML (de)serialisation of trajectory groups (parity: reference
``src/art/utils/trajectory_logging.py:9-84``).  Token log-probs are dropped on write."""
from __future__ import annotations

from typing import Any

import yaml
from openai.types.chat.chat_completion import Choice

from ..trajectories import Trajectory, TrajectoryGroup


def message_or_choice_to_dict(item) -> dict[str, Any]:
    d = dict(item) if isinstance(item, dict) else item.to_dict()
    d.pop("logprobs", None)
    return d


def trajectory_to_dict(t: Trajectory) -> dict[str, Any]:
    return {
        "reward": t.reward,
        "metrics": dict(t.metrics),
        "metadata": dict(t.metadata),
        "messages_and_choices": [message_or_choice_to_dict(m) for m in t.messages_and_choices],
        "logs": list(t.logs),
    }


def trajectory_group_to_dict(g: TrajectoryGroup) -> dict[str, Any]:
    return {"trajectories": [trajectory_to_dict(t) for t in g.trajectories if isinstance(t, Trajectory)],
            "metadata": dict(g.metadata)}


def serialize_trajectory_groups(groups: list[TrajectoryGroup]) -> str:
    return yaml.safe_dump([trajectory_group_to_dict(g) for g in groups], sort_keys=True)


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


def deserialize_trajectory_groups(text: str) -> list[TrajectoryGroup]:
    return [dict_to_trajectory_group(g) for g in (yaml.safe_load(text) or [])]
