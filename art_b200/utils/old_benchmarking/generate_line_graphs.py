"""One line graph per metric, written under ``{art_path}/{project}/benchmarks`` (parity: reference
``src/art/utils/old_benchmarking/generate_line_graphs.py:11-70``): the ``line_graph_keys`` models are lines over step
index (or over the time their steps were recorded), the ``comparison_keys`` models are dashed horizontal lines at
their last step's value.  The files are SVG (``benchmarking/charts/svg.py``); returns their paths.
"""
from __future__ import annotations

import os
from datetime import datetime
from typing import Literal

from ..benchmarking.charts.svg import PALETTE, SvgFigure, nice_ticks
from ..output_dirs import get_default_art_path
from .load_benchmarked_models import load_benchmarked_models
from .types import BenchmarkedModelKey


def _seconds(ts: str, origin: datetime) -> float:
    return (datetime.fromisoformat(ts) - origin).total_seconds()


def generate_line_graphs(project: str, line_graph_keys: list[BenchmarkedModelKey],
                         comparison_keys: list[BenchmarkedModelKey], metrics: list[str] | None = None,
                         x_axis_metric: Literal["step", "time"] = "step", api_path: str | None = None) -> list[str]:
    metrics = list(metrics) if metrics is not None else ["reward"]
    api_path = api_path or get_default_art_path()
    out_dir = os.path.join(api_path, project, "benchmarks")
    os.makedirs(out_dir, exist_ok=True)
    lines = load_benchmarked_models(project, line_graph_keys, metrics, api_path)
    if x_axis_metric == "time":
        kept = []
        for m in lines:
            if all(s.recorded_at is not None for s in m.steps):
                kept.append(m)
            else:
                print(f"WARNING: Model {m.model_key} is missing a recorded_at time for a step, removing from line graph models")
        lines = kept
    comparisons = load_benchmarked_models(project, comparison_keys, metrics, api_path) if comparison_keys else []
    paths = []
    for metric in metrics:
        curves = []
        for m in lines:
            if x_axis_metric == "time":
                origin = datetime.fromisoformat(m.steps[0].recorded_at)
                xs = [_seconds(s.recorded_at, origin) for s in m.steps]
            else:
                xs = [float(s.index) for s in m.steps]
            pts = [(x, s.metrics[metric]) for x, s in zip(xs, m.steps) if metric in s.metrics]
            curves.append((f"{m.model_key.model} {m.model_key.split}", pts))
        levels = [(f"{m.model_key.model} {m.model_key.split}", m.steps[-1].metrics[metric])
                  for m in comparisons if m.steps and metric in m.steps[-1].metrics]
        xs_all = [x for _, pts in curves for x, _ in pts] or [0.0]
        ys_all = [y for _, pts in curves for _, y in pts] + [y for _, y in levels] or [0.0]
        fig = SvgFigure()
        y_ticks = nice_ticks(min(ys_all), max(ys_all))
        fig.set_limits(min(xs_all), max(xs_all), y_ticks[0], y_ticks[-1])
        fig.axes(x_ticks=nice_ticks(fig.x0, fig.x1), y_ticks=y_ticks, x_label=x_axis_metric, y_label=metric, title=metric)
        legend = []
        for i, (label, pts) in enumerate(curves):
            color = PALETTE[i % len(PALETTE)]
            if pts:
                fig.polyline([(fig.px(x), fig.py(y)) for x, y in pts], color)
                fig.circle(fig.px(pts[-1][0]), fig.py(pts[-1][1]), 3, color)      # a dot on the newest point only
            legend.append((label, color))
        for label, y in levels:
            fig.line(fig.px(fig.x0), fig.py(y), fig.px(fig.x1), fig.py(y), color="#000", dash="6 4")
            fig.text(fig.px(fig.x1) - 4, fig.py(y) - 4, label, size=9, anchor="end", color="#000")
        fig.legend(legend, "lower right")
        stamp = datetime.now().strftime("%Y-%m-%d_%H-%M-%S.%f")[:-3]
        paths.append(fig.savefig(os.path.join(out_dir, f"{stamp}_{metric}_line_graph.svg")))
    return paths
