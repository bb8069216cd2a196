"""A small SVG figure writer for the benchmark charts.

The reference draws its charts with matplotlib + seaborn
(``src/art/utils/benchmarking/charts/*.py``); both are optional here.  The charts need only
axes, poly-lines, bars, hatching and text, which is little enough to emit as SVG directly, so
they work (and are tested) on a machine with neither library installed.  A figure renders
inline in notebooks through ``_repr_svg_``.
"""
from __future__ import annotations

import math
from xml.sax.saxutils import escape

PALETTE = ["#e67e22", "#2980b9", "#27ae60", "#8e44ad", "#c0392b", "#16a085", "#7f8c8d", "#d35400"]


def nice_ticks(lo: float, hi: float, n: int = 5) -> list[float]:
    """Round tick positions covering [lo, hi] (1-2-5 steps)."""
    if not math.isfinite(lo) or not math.isfinite(hi):
        return [0.0, 1.0]
    if hi <= lo:
        hi = lo + (abs(lo) or 1.0)
    raw = (hi - lo) / max(1, n)
    mag = 10 ** math.floor(math.log10(raw))
    step = next(m * mag for m in (1, 2, 5, 10) if m * mag >= raw)
    first = math.floor(lo / step) * step
    ticks, t = [], first
    while t <= hi + step * 1e-9:
        ticks.append(round(t, 10))
        t += step
    if ticks[-1] < hi - step * 1e-9:
        ticks.append(round(ticks[-1] + step, 10))
    return ticks


class SvgFigure:
    """Canvas with one plot area; data coordinates are mapped by :meth:`set_limits`."""

    def __init__(self, width: int = 720, height: int = 480, margins=(70, 30, 50, 60)):
        self.width, self.height = width, height
        self.left, self.right, self.top, self.bottom = margins
        self.x0 = self.x1 = self.y0 = self.y1 = 0.0
        self.set_limits(0, 1, 0, 1)
        self.parts: list[str] = []
        self.defs: list[str] = []
        self.texts: list[str] = []          # every string drawn, for tests and accessibility

    # -- coordinates ----------------------------------------------------------------------------
    def set_limits(self, x0: float, x1: float, y0: float, y1: float) -> None:
        self.x0, self.x1 = (x0, x1) if x1 > x0 else (x0, x0 + 1)
        self.y0, self.y1 = (y0, y1) if y1 > y0 else (y0, y0 + 1)

    def px(self, x: float) -> float:
        return self.left + (x - self.x0) / (self.x1 - self.x0) * (self.width - self.left - self.right)

    def py(self, y: float) -> float:
        return self.height - self.bottom - (y - self.y0) / (self.y1 - self.y0) * (self.height - self.top - self.bottom)

    # -- primitives (pixel coordinates) ---------------------------------------------------------
    def line(self, xa, ya, xb, yb, color="#333", width=1.0, dash: str | None = None) -> None:
        d = f' stroke-dasharray="{dash}"' if dash else ""
        self.parts.append(f'<line x1="{xa:.1f}" y1="{ya:.1f}" x2="{xb:.1f}" y2="{yb:.1f}" stroke="{color}" '
                          f'stroke-width="{width}"{d}/>')

    def polyline(self, pts, color, width=2.0) -> None:
        s = " ".join(f"{x:.1f},{y:.1f}" for x, y in pts)
        self.parts.append(f'<polyline points="{s}" fill="none" stroke="{color}" stroke-width="{width}"/>')

    def circle(self, x, y, r, color) -> None:
        self.parts.append(f'<circle cx="{x:.1f}" cy="{y:.1f}" r="{r}" fill="{color}"/>')

    def rect(self, x, y, w, h, fill, stroke="none", hatch: bool = False) -> None:
        if hatch:
            pid = f"hatch{len(self.defs)}"
            self.defs.append(f'<pattern id="{pid}" width="8" height="8" patternUnits="userSpaceOnUse" '
                             f'patternTransform="rotate(45)"><rect width="8" height="8" fill="{fill}" fill-opacity="0.45"/>'
                             f'<line x1="0" y1="0" x2="0" y2="8" stroke="{fill}" stroke-width="3"/></pattern>')
            fill = f"url(#{pid})"
        self.parts.append(f'<rect x="{x:.1f}" y="{y:.1f}" width="{max(w, 0):.1f}" height="{max(h, 0):.1f}" fill="{fill}" '
                          f'stroke="{stroke}"/>')

    def text(self, x, y, s: str, size=12, anchor="middle", color="#222", weight="normal", rotate: float | None = None) -> None:
        self.texts.append(s)
        tr = f' transform="rotate({rotate} {x:.1f} {y:.1f})"' if rotate is not None else ""
        self.parts.append(f'<text x="{x:.1f}" y="{y:.1f}" font-size="{size}" text-anchor="{anchor}" fill="{color}" '
                          f'font-family="Helvetica, Arial, sans-serif" font-weight="{weight}"{tr}>{escape(s)}</text>')

    # -- composites -----------------------------------------------------------------------------
    def axes(self, x_ticks=None, y_ticks=None, x_label=None, y_label=None, title=None, x_tick_labels=None,
             y_fmt=lambda v: f"{v:g}") -> None:
        bx0, bx1, by0, by1 = self.px(self.x0), self.px(self.x1), self.py(self.y0), self.py(self.y1)
        self.line(bx0, by0, bx1, by0)
        self.line(bx0, by0, bx0, by1)
        for i, t in enumerate(x_ticks or []):
            self.line(self.px(t), by0, self.px(t), by0 + 4)
            self.text(self.px(t), by0 + 18, x_tick_labels[i] if x_tick_labels else f"{t:g}", size=11)
        for t in y_ticks or []:
            self.line(bx0 - 4, self.py(t), bx0, self.py(t))
            self.text(bx0 - 8, self.py(t) + 4, y_fmt(t), size=11, anchor="end")
        if x_label:
            self.text((bx0 + bx1) / 2, self.height - 12, x_label, size=13)
        if y_label:
            self.text(18, (by0 + by1) / 2, y_label, size=13, rotate=-90)
        if title:
            self.text(self.width / 2, 20, title, size=15, weight="bold")

    def legend(self, entries: list[tuple[str, str]], loc: str = "lower right") -> None:
        """``entries``: (label, colour).  ``loc``: "lower right", "upper left", ..."""
        if not entries:
            return
        w = 30 + 7 * max(len(e[0]) for e in entries)
        h = 8 + 18 * len(entries)
        x = self.width - self.right - w - 8 if "right" in loc else self.left + 8
        y = self.height - self.bottom - h - 8 if "lower" in loc else self.top + 8
        self.rect(x, y, w, h, "#ffffff", stroke="#bbb")
        for i, (label, color) in enumerate(entries):
            cy = y + 14 + 18 * i
            self.line(x + 6, cy - 4, x + 22, cy - 4, color=color, width=3)
            self.text(x + 27, cy, label, size=11, anchor="start")

    # -- output ---------------------------------------------------------------------------------
    def to_svg(self) -> str:
        defs = f"<defs>{''.join(self.defs)}</defs>" if self.defs else ""
        return (f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.width}" height="{self.height}" '
                f'viewBox="0 0 {self.width} {self.height}"><rect width="100%" height="100%" fill="#ffffff"/>{defs}'
                + "".join(self.parts) + "</svg>")

    def _repr_svg_(self) -> str:
        return self.to_svg()

    def savefig(self, path: str) -> str:
        with open(path, "w") as f:
            f.write(self.to_svg())
        return path
