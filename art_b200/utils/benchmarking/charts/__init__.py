"""Benchmark charts (parity: reference ``src/art/utils/benchmarking/charts``).

``training_progress_table`` / ``comparison_table`` do the aggregation and need only pandas;
``training_progress_chart`` / ``percentage_comparison_bar_chart`` draw them and need matplotlib
(optional, imported lazily, Agg backend: no display or graphics API involved).
"""
from __future__ import annotations

from ..filter_model_split import filter_rename_model_split
from ..types import BenchmarkModelKey


def _keys(models) -> list[BenchmarkModelKey]:
    return [m if isinstance(m, BenchmarkModelKey) else BenchmarkModelKey(m) for m in models]


def training_progress_table(df, metric_name: str, models, perfect_score: float | None = None):
    """Mean of ``metric_name`` per (model, step) for the requested models/splits."""
    import pandas as pd

    col = metric_name if metric_name in df.columns else f"metric_{metric_name}"
    parts = []
    for key in _keys(models):
        sub = filter_rename_model_split(df, key)
        if len(sub):
            parts.append(sub.groupby(["model", "step"], as_index=False)[col].mean())
    out = pd.concat(parts) if parts else pd.DataFrame(columns=["model", "step", col])
    return out.rename(columns={col: metric_name})


def comparison_table(df, metric_name: str, models):
    """Per model: mean of the metric at the first and at the last logged step."""
    prog = training_progress_table(df, metric_name, models)
    rows = []
    for model, g in prog.groupby("model"):
        g = g.sort_values("step")
        rows.append({"model": model, "first": g[metric_name].iloc[0], "last": g[metric_name].iloc[-1],
                     "improvement": g[metric_name].iloc[-1] - g[metric_name].iloc[0]})
    import pandas as pd

    return pd.DataFrame(rows)


def _plt():
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt

        return plt
    except ImportError as e:
        raise RuntimeError("charts need matplotlib, which is not installed") from e


def training_progress_chart(df, metric_name: str, models, title: str | None = None, perfect_score: float | None = None,
                            y_label: str | None = None, path: str | None = None):
    plt = _plt()
    prog = training_progress_table(df, metric_name, models)
    fig, ax = plt.subplots(figsize=(8, 5))
    for model, g in prog.groupby("model"):
        g = g.sort_values("step")
        ax.plot(g["step"], g[metric_name], marker="o", label=model)
    if perfect_score is not None:
        ax.axhline(perfect_score, linestyle="--", color="gray")
    ax.set_xlabel("Step")
    ax.set_ylabel(y_label or metric_name)
    ax.set_title(title or metric_name)
    ax.legend()
    if path:
        fig.savefig(path)
    return fig


def percentage_comparison_bar_chart(df, metric_name: str, models, title: str | None = None, path: str | None = None):
    plt = _plt()
    table = comparison_table(df, metric_name, models)
    fig, ax = plt.subplots(figsize=(8, 5))
    bars = ax.bar(table["model"], table["last"] * 100)
    for bar, (_, row) in zip(bars, table.iterrows()):
        label = f"{row['last'] * 100:.0f}%"
        if row["improvement"] > 0:
            label += f"\nRL +{row['improvement'] * 100:.0f}%"
        ax.text(bar.get_x() + bar.get_width() / 2, bar.get_height(), label, ha="center", va="bottom")
    ax.set_ylabel(f"{metric_name} (%)")
    ax.set_title(title or metric_name)
    if path:
        fig.savefig(path)
    return fig
