"""Load per-step metric averages of logged models (parity: reference
``src/art/utils/old_benchmarking/load_benchmarked_models.py:18-108``).

For every requested (model, split) the steps' trajectory files are read, each metric is averaged
inside a group and then over groups (``reward`` counts as a metric), ``reward_std_dev`` is added, and
the wall-clock time of the step is taken from the newest ``history.jsonl`` row of that step that has
a ``recorded_at`` field.  The caller's keys are not modified.
"""
from __future__ import annotations

import json
import os

from ..output_dirs import get_default_art_path, get_output_dir_from_model_properties, get_trajectories_split_dir
from ..trajectory_logging import deserialize_trajectory_groups
from .calculate_step_metrics import calculate_step_std_dev
from .types import BenchmarkedModel, BenchmarkedModelKey, BenchmarkedModelStep


def _logged_steps(split_dir: str) -> list[int]:
    steps = []
    for name in os.listdir(split_dir):
        stem, ext = os.path.splitext(name)
        if ext == ".yaml" and stem.isdigit():
            steps.append(int(stem))
    return sorted(steps)


def _history_times(model_dir: str) -> dict[int, str]:
    times: dict[int, str] = {}
    path = os.path.join(model_dir, "history.jsonl")
    if not os.path.exists(path):
        return times
    with open(path) as f:
        for line in f:
            try:
                row = json.loads(line)
            except json.JSONDecodeError:
                continue
            if "recorded_at" in row and "step" in row:
                times[int(row["step"])] = row["recorded_at"]     # later rows win
    return times


def load_benchmarked_models(project: str, benchmark_keys: list[BenchmarkedModelKey], metrics: list[str] | None = None,
                            api_path: str | None = None) -> list[BenchmarkedModel]:
    metrics = list(metrics) if metrics is not None else ["reward"]
    api_path = api_path or get_default_art_path()
    out = []
    for key in benchmark_keys:
        model_dir = get_output_dir_from_model_properties(project=project, name=key.model, art_path=api_path)
        split_dir = get_trajectories_split_dir(model_dir, key.split)
        logged = _logged_steps(split_dir) if os.path.isdir(split_dir) else []
        if not logged:
            raise FileNotFoundError(f"no logged trajectories for {key.model} / {key.split} under {split_dir}")
        last = logged[-1]
        wanted = logged if key.step_indices is None else [last + 1 + i if i < 0 else i for i in key.step_indices]
        times = _history_times(model_dir)
        model = BenchmarkedModel(BenchmarkedModelKey(key.model, key.split, list(wanted)))
        for index in wanted:
            with open(os.path.join(split_dir, f"{index:04d}.yaml")) as f:
                groups = deserialize_trajectory_groups(f.read())
            step = BenchmarkedModelStep(index, recorded_at=times.get(index))
            for metric in metrics:
                group_means = []
                for g in groups:
                    vals = [t.reward if metric == "reward" and "reward" not in t.metrics else t.metrics[metric]
                            for t in g.trajectories
                            if not isinstance(t, BaseException) and (metric in t.metrics or metric == "reward")]
                    if vals:
                        group_means.append(sum(vals) / len(vals))
                if group_means:
                    step.metrics[metric] = sum(group_means) / len(group_means)
            step.metrics["reward_std_dev"] = calculate_step_std_dev(groups)
            model.steps.append(step)
        out.append(model)
    return out
