"""Flatten logged trajectory YAML files into a table (parity: reference
``src/art/utils/benchmarking/load_trajectories.py:18-197``).

Layout read: ``{art_path}/{project}/models/{model}/trajectories/{split}/{step:04d}.yaml``.
One row per trajectory with fixed columns ``model, split, step, reward, group_number, messages,
logs`` plus ``metric_*`` and ``metadata_*`` columns.  The table is a pandas DataFrame (polars, which
the reference uses, is optional: ``as_polars=True`` converts when it is installed).
"""
from __future__ import annotations

import os
from pathlib import Path

import yaml

from ..output_dirs import get_default_art_path, get_models_dir, get_trajectories_dir


def load_trajectory_rows(project_name: str, models: list[str] | None = None, art_path: str | None = None,
                         debug: bool = False) -> list[dict]:
    art_path = art_path or get_default_art_path()
    root = Path(get_models_dir(project_name, art_path))
    rows: list[dict] = []
    group_number = 0
    if not root.exists():
        return rows
    for model_dir in sorted(p for p in root.iterdir() if p.is_dir()):
        if models is not None and model_dir.name not in models:
            continue
        traj_root = Path(get_trajectories_dir(str(model_dir)))
        if not traj_root.exists():
            continue
        for split_dir in sorted(p for p in traj_root.iterdir() if p.is_dir()):
            for f in sorted(split_dir.glob("*.yaml")):
                try:
                    step = int(f.stem)
                except ValueError:
                    continue
                try:
                    groups = yaml.safe_load(f.read_text()) or []
                except yaml.YAMLError as e:
                    if debug:
                        print(f"skipping unreadable {f}: {e}")
                    continue
                for group in groups:
                    group_number += 1
                    for t in group.get("trajectories", []):
                        row = {"model": model_dir.name, "split": split_dir.name, "step": step,
                               "reward": t.get("reward"), "group_number": group_number,
                               "messages": t.get("messages_and_choices"), "logs": t.get("logs")}
                        for k, v in (t.get("metrics") or {}).items():
                            row[f"metric_{k}"] = v
                        for k, v in {**(group.get("metadata") or {}), **(t.get("metadata") or {})}.items():
                            row[f"metadata_{k}"] = v
                        rows.append(row)
    return rows


async def load_trajectories(project_name: str, models: list[str] | None = None, debug: bool = False,
                            art_path: str | None = None, as_polars: bool = False):
    import pandas as pd

    df = pd.DataFrame(load_trajectory_rows(project_name, models, art_path, debug))
    if as_polars:
        import polars as pl  # optional

        return pl.from_pandas(df)
    return df
