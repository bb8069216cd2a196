"""One table row per (model, split, step) with the requested metric means (parity: reference
``src/art/utils/old_benchmarking/generate_comparison_table.py:6-27``)."""
from __future__ import annotations

from .load_benchmarked_models import load_benchmarked_models
from .types import BenchmarkedModelKey


def generate_comparison_table(project: str, benchmark_keys: list[BenchmarkedModelKey], metrics: list[str] | None = None,
                              api_path: str | None = None):
    import pandas as pd

    metrics = list(metrics) if metrics is not None else ["reward"]
    rows = []
    for model in load_benchmarked_models(project, benchmark_keys, metrics, api_path):
        for step in model.steps:
            row = {"Model": model.model_key.model, "Split": model.model_key.split, "Step": f"{step.index:04d}"}
            for m in metrics:
                row[m] = step.metrics.get(m, "N/A")
            rows.append(row)
    return pd.DataFrame(rows, columns=["Model", "Split", "Step"] + metrics)
