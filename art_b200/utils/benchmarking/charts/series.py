"""Aggregations behind the benchmark charts (pandas only; the drawing is in the chart modules)."""
from __future__ import annotations

from ..filter_model_split import filter_rename_model_split
from ..types import BenchmarkModelKey


def resolve_metric_column(df, metric_name: str) -> str:
    col = metric_name if metric_name in df.columns else f"metric_{metric_name}"
    if col not in df.columns:
        raise ValueError(f"Column '{col}' not found in DataFrame. Available columns: {list(df.columns)}")
    return col


def as_keys(models) -> list[BenchmarkModelKey] | None:
    if models is None:
        return None
    return [m if isinstance(m, BenchmarkModelKey) else BenchmarkModelKey(m) for m in models]


def select_models(df, models):
    """Rows of the requested models/splits (renamed to their display names) and the plotting order.

    Without an explicit list: trained models (several distinct steps) first, prompted comparison models (one step)
    after them, each group alphabetically, as the reference orders them
    (``charts/training_progress_chart.py:84-103``)."""
    import pandas as pd

    keys = as_keys(models)
    if keys is not None:
        parts = [filter_rename_model_split(df, k) for k in keys]
        out = pd.concat(parts) if parts else df.iloc[0:0]
        order = [k.display_name for k in keys]
    else:
        out = df
        n_steps = out.groupby("model")["step"].nunique()
        order = sorted(m for m, n in n_steps.items() if n > 1) + sorted(m for m, n in n_steps.items() if n <= 1)
    if len(out) == 0:
        raise ValueError("No rows left after applying the split filter. Check your 'split' argument or the DataFrame contents.")
    return out, order


def progress_series(df, metric_name: str, models=None) -> dict[str, list[tuple[int, float]]]:
    """model -> [(step, mean metric)] sorted by step, in plotting order."""
    col = resolve_metric_column(df, metric_name)
    sub, order = select_models(df, models)
    agg = sub.groupby(["model", "step"], as_index=False)[col].mean().sort_values("step")
    series: dict[str, list[tuple[int, float]]] = {}
    for name in order:
        rows = agg[agg["model"] == name]
        if len(rows):
            series[name] = [(int(s), float(v)) for s, v in zip(rows["step"], rows[col]) if v == v]
    return series


def first_last(df, metric_name: str, models=None) -> list[dict]:
    """Per model: metric mean at its first and last step; ``trained`` is False for single-step models."""
    out = []
    for name, pts in progress_series(df, metric_name, models).items():
        if not pts:
            continue
        out.append({"model": name, "first": pts[0][1], "last": pts[-1][1], "trained": len(pts) > 1,
                    "improvement": pts[-1][1] - pts[0][1]})
    return out
