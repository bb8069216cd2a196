"""Bar chart comparing models on a 0..1 metric shown as percentages.

Parity: reference ``src/art/utils/benchmarking/charts/percentage_comparison_bar_chart.py:6-251``:
a trained model is a stacked bar (solid base = score at its first step, hatched segment = change by
its last step) annotated ``RL +N%`` (relative improvement over the first step, as in the
reference's published charts), a model evaluated once is a single solid bar; every bar carries its
final percentage.  Drawn as SVG (``svg.py``).
"""
from __future__ import annotations

from .series import first_last
from .svg import PALETTE, SvgFigure, nice_ticks


def rl_improvement_label(first: float, last: float) -> str | None:
    """``RL +52%``-style label: change of the last score relative to the first one."""
    if first <= 0 or last == first:
        return None
    pct = (last - first) / first * 100.0
    return f"RL {'+' if pct >= 0 else '-'}{abs(pct):.0f}%"


def percentage_comparison_bar_chart(df, metric_name: str, models=None, title: str | None = None,
                                    y_label: str | None = None, perfect_score: float | None = None,
                                    path: str | None = None) -> SvgFigure:
    rows = first_last(df, metric_name, models)
    fig = SvgFigure()
    top = max([max(r["first"], r["last"]) for r in rows] + ([perfect_score] if perfect_score is not None else []) + [1e-9])
    y_ticks = nice_ticks(0.0, top * 100.0 * 1.12)
    n = max(1, len(rows))
    fig.set_limits(0, n, 0, y_ticks[-1])
    fig.axes(x_ticks=[i + 0.5 for i in range(len(rows))], x_tick_labels=[r["model"] for r in rows], y_ticks=y_ticks,
             y_label=y_label, title=title or f"{metric_name} (%)", y_fmt=lambda v: f"{v:g}%")
    for i, r in enumerate(rows):
        color = PALETTE[0] if r["trained"] else PALETTE[6]
        xa, xb = fig.px(i + 0.2), fig.px(i + 0.8)
        lo, hi = min(r["first"], r["last"]) * 100, max(r["first"], r["last"]) * 100
        base = r["first"] * 100 if r["trained"] and r["last"] >= r["first"] else r["last"] * 100
        fig.rect(xa, fig.py(base), xb - xa, fig.py(0) - fig.py(base), color)
        if r["trained"] and hi > lo:
            fig.rect(xa, fig.py(hi), xb - xa, fig.py(lo) - fig.py(hi), color, hatch=True)
        fig.text((xa + xb) / 2, fig.py(max(hi, base)) - 6, f"{r['last'] * 100:.0f}%", size=12, weight="bold")
        label = rl_improvement_label(r["first"], r["last"]) if r["trained"] else None
        if label:
            fig.text((xa + xb) / 2, fig.py(max(hi, base)) - 22, label, size=11, color=color)
    if perfect_score is not None:
        y = fig.py(perfect_score * 100)
        fig.line(fig.px(0), y, fig.px(n), y, color="#999", dash="2 3")
        fig.text(fig.px(0) + 6, y - 5, "Perfect score", size=10, anchor="start", color="#777")
    fig.rows = rows
    if path:
        fig.savefig(path)
    return fig
