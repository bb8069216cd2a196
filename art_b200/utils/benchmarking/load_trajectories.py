"""Flatten logged trajectory YAML files into a table (parity: reference
``src/art/utils/benchmarking/load_trajectories.py:18-197``).

Layout read: ``{art_path}/{project}/models/{model}/trajectories/{split}/{step:04d}.yaml``.
One row per trajectory with fixed columns ``model, split, step, reward, group_number, messages,
logs`` plus ``metric_*`` (float) and ``metadata_*`` (string) columns; ``messages`` is the dialogue
with a ``trainable`` flag per entry (True for sampled choices).  The table is a pandas DataFrame
(polars, which the reference uses, is optional: ``as_polars=True`` converts when it is installed).

Parsing a long run's YAML is slow, so rows are cached in a SQLite file under
``{art_path}/{project}/.benchmark_cache.sqlite`` keyed by file path; an entry is reused only while
the file's size and modification time are unchanged (the reference memoises the whole call with
``panza.SQLiteCache`` and therefore never sees files written after the first call).
"""
from __future__ import annotations

import json
import os
import sqlite3
from pathlib import Path

import yaml

from ..output_dirs import get_default_art_path, get_models_dir, get_trajectories_dir


def _flatten_messages(entries) -> list[dict]:
    out = []
    for m in entries or []:
        if isinstance(m, dict) and "message" in m:      # a sampled Choice: its message is what was trained on
            out.append({**(m["message"] or {}), "trainable": True})
        elif isinstance(m, dict):
            out.append({**m, "trainable": False})
    return out


def _rows_of_file(path: Path) -> list[dict]:
    """Rows of one YAML file without the columns that depend on where the file sits (model, split, step, group_number);
    ``group_index`` numbers the groups inside the file."""
    groups = yaml.safe_load(path.read_text()) or []
    rows = []
    for gi, group in enumerate(groups):
        gmeta = group.get("metadata") or {}
        for t in group.get("trajectories", []):
            row = {"group_index": gi, "reward": t.get("reward"), "messages": _flatten_messages(t.get("messages_and_choices")),
                   "logs": t.get("logs")}
            for k, v in (t.get("metrics") or {}).items():
                row[f"metric_{k}"] = v
            for k, v in {**gmeta, **(t.get("metadata") or {})}.items():     # trajectory metadata wins
                row[f"metadata_{k}"] = str(v)
            rows.append(row)
    return rows


class _FileCache:
    """path -> (size, mtime_ns, rows as JSON); any error falls back to parsing."""

    def __init__(self, db_path: str | None):
        self.db = None
        if db_path:
            try:
                os.makedirs(os.path.dirname(db_path), exist_ok=True)
                self.db = sqlite3.connect(db_path)
                self.db.execute("create table if not exists files (path text primary key, size int, mtime int, rows text)")
            except (sqlite3.Error, OSError):
                self.db = None

    def rows(self, path: Path) -> list[dict]:
        st = path.stat()
        if self.db is not None:
            try:
                hit = self.db.execute("select size, mtime, rows from files where path = ?", (str(path),)).fetchone()
                if hit and hit[0] == st.st_size and hit[1] == st.st_mtime_ns:
                    return json.loads(hit[2])
            except (sqlite3.Error, ValueError):
                pass
        rows = _rows_of_file(path)
        if self.db is not None:
            try:
                self.db.execute("insert or replace into files values (?, ?, ?, ?)",
                                (str(path), st.st_size, st.st_mtime_ns, json.dumps(rows, default=str)))
            except (sqlite3.Error, TypeError):
                pass
        return rows

    def close(self) -> None:
        if self.db is not None:
            try:
                self.db.commit()
                self.db.close()
            except sqlite3.Error:
                pass


def load_trajectory_rows(project_name: str, models: list[str] | None = None, art_path: str | None = None,
                         debug: bool = False, use_cache: bool = True) -> list[dict]:
    art_path = art_path or get_default_art_path()
    root = Path(get_models_dir(project_name, art_path))
    rows: list[dict] = []
    if not root.exists():
        return rows
    cache = _FileCache(os.path.join(art_path, project_name, ".benchmark_cache.sqlite") if use_cache else None)
    group_number = 0
    try:
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
                    if debug:
                        print(f"Processing {f}")
                    try:
                        file_rows = cache.rows(f)
                    except yaml.YAMLError as e:
                        if debug:
                            print(f"skipping unreadable {f}: {e}")
                        continue
                    n_groups = 0
                    for r in file_rows:
                        r = dict(r)
                        gi = r.pop("group_index", 0)
                        n_groups = max(n_groups, gi + 1)
                        rows.append({"model": model_dir.name, "split": split_dir.name, "step": step,
                                     "reward": r.pop("reward"), "group_number": group_number + gi + 1, **r})
                    group_number += n_groups
    finally:
        cache.close()
    return rows


async def load_trajectories(project_name: str, models: list[str] | None = None, debug: bool = False,
                            art_path: str | None = None, as_polars: bool = False, use_cache: bool = True):
    import pandas as pd

    rows = load_trajectory_rows(project_name, models, art_path, debug, use_cache)
    fixed = ["model", "split", "step", "reward", "group_number", "messages", "logs"]
    extra = sorted({k for r in rows for k in r} - set(fixed))
    df = pd.DataFrame(rows, columns=fixed + extra)
    for c in extra:
        if c.startswith("metric_"):
            df[c] = pd.to_numeric(df[c], errors="coerce")
    if as_polars:
        import polars as pl  # optional

        return pl.from_pandas(df)
    return df
