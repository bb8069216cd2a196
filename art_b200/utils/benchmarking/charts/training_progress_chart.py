"""Line chart of a metric over training steps, one line per model.

Parity: reference ``src/art/utils/benchmarking/charts/training_progress_chart.py:9-265``: trained
models are lines with a marker on the last point, models evaluated at a single step (prompted
comparison models) are dashed horizontal lines across the plot labelled at the right edge, an
optional "Perfect score" reference line, legend location as an argument.  Drawn as SVG (see
``svg.py``); returns the figure object (``.savefig(path)``, ``_repr_svg_`` for notebooks).
"""
from __future__ import annotations

from .series import progress_series
from .svg import PALETTE, SvgFigure, nice_ticks


def training_progress_chart(df, metric_name: str, models=None, title: str | None = None, x_label: str | None = None,
                            y_label: str | None = None, perfect_score: float | None = None,
                            legend_loc: str | None = "lower right", path: str | None = None) -> SvgFigure:
    series = progress_series(df, metric_name, models)
    trained = {m: p for m, p in series.items() if len(p) > 1}
    single = {m: p for m, p in series.items() if len(p) == 1}
    steps = [s for p in series.values() for s, _ in p] or [0]
    values = [v for p in series.values() for _, v in p] + ([perfect_score] if perfect_score is not None else [])
    fig = SvgFigure()
    y_ticks = nice_ticks(min(values + [0.0]), max(values))
    x_lo, x_hi = min(steps), max(steps)
    fig.set_limits(x_lo, x_hi if x_hi > x_lo else x_lo + 1, y_ticks[0], y_ticks[-1])
    fig.axes(x_ticks=[t for t in nice_ticks(x_lo, max(x_hi, x_lo + 1)) if x_lo <= t <= max(x_hi, x_lo + 1) and t == int(t)],
             y_ticks=y_ticks, x_label="Step" if x_label is None else x_label, y_label=y_label,
             title=title or f"{metric_name} over training")
    legend = []
    for i, (name, pts) in enumerate(trained.items()):
        color = PALETTE[i % len(PALETTE)]
        fig.polyline([(fig.px(s), fig.py(v)) for s, v in pts], color)
        fig.circle(fig.px(pts[-1][0]), fig.py(pts[-1][1]), 4, color)
        legend.append((name, color))
    for name, pts in single.items():
        y = fig.py(pts[0][1])
        fig.line(fig.px(fig.x0), y, fig.px(fig.x1), y, color="#555", dash="6 4")
        fig.text(fig.px(fig.x1) - 4, y - 4, name, size=10, anchor="end", color="#555")
    if perfect_score is not None:
        y = fig.py(perfect_score)
        fig.line(fig.px(fig.x0), y, fig.px(fig.x1), y, color="#999", dash="2 3")
        fig.text(fig.px(fig.x0) + 6, y - 5, "Perfect score", size=10, anchor="start", color="#777")
    if legend_loc:
        fig.legend(legend, legend_loc)
    fig.series = series          # the plotted numbers, for callers and tests
    if path:
        fig.savefig(path)
    return fig
