"""A dependency-free line / scatter chart writer (plain SVG), shared by the analysis scripts of this package.

The reference draws its figures with matplotlib (`plots/*.py`); the image built here carries no plotting library, so the
scripts compute their tables with numpy / scipy and hand the points to this writer."""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

COLORS = ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf"]


def _ticks(lo: float, hi: float, log: bool) -> List[float]:
    if log:
        a, b = int(np.floor(lo)), int(np.ceil(hi))
        return [float(v) for v in range(a, b + 1) if lo - 1e-9 <= v <= hi + 1e-9] or [lo, hi]
    span = hi - lo
    if span <= 0:
        return [lo]
    step = 10 ** np.floor(np.log10(span / 5))
    for m in (1, 2, 5, 10):
        if span / (step * m) <= 6:
            step *= m
            break
    first = np.ceil(lo / step) * step
    return [float(v) for v in np.arange(first, hi + 1e-12, step)]


def line_chart(path: str, series: Iterable[Dict], xlabel: str, ylabel: str, title: str = "", logx: bool = False,
               logy: bool = False, width: int = 900, height: int = 600) -> None:
    """``series``: dicts with ``name``, ``x``, ``y`` and optionally ``style`` ("line", "points", "both"; default "both"),
    ``curve_x`` / ``curve_y`` (a fitted curve drawn under the points) and ``star`` (an (x, y) optimum marker)."""
    series = [s for s in series if len(s["x"])]
    m = 75
    tx = (lambda v: np.log10(np.asarray(v, dtype=np.float64))) if logx else (lambda v: np.asarray(v, dtype=np.float64))
    ty = (lambda v: np.log10(np.asarray(v, dtype=np.float64))) if logy else (lambda v: np.asarray(v, dtype=np.float64))
    xs = np.concatenate([tx(s["x"]) for s in series] + [tx(s["curve_x"]) for s in series if "curve_x" in s])
    ys = np.concatenate([ty(s["y"]) for s in series] + [ty(s["curve_y"]) for s in series if "curve_y" in s])
    xs, ys = xs[np.isfinite(xs)], ys[np.isfinite(ys)]
    x0, x1 = float(xs.min()), float(xs.max())
    y0, y1 = float(ys.min()), float(ys.max())
    padx, pady = 0.04 * (x1 - x0 or 1.0), 0.06 * (y1 - y0 or 1.0)
    x0, x1, y0, y1 = x0 - padx, x1 + padx, y0 - pady, y1 + pady
    px = lambda v: m + (tx(v) - x0) / (x1 - x0) * (width - 2 * m)
    py = lambda v: height - m - (ty(v) - y0) / (y1 - y0) * (height - 2 * m)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="13">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<line x1="{m}" y1="{height - m}" x2="{width - m}" y2="{height - m}" stroke="black"/>',
           f'<line x1="{m}" y1="{m}" x2="{m}" y2="{height - m}" stroke="black"/>',
           f'<text x="{width / 2}" y="{height - 22}" text-anchor="middle">{xlabel}{" (log scale)" if logx else ""}</text>',
           f'<text x="22" y="{height / 2}" text-anchor="middle" transform="rotate(-90 22 {height / 2})">{ylabel}'
           f'{" (log scale)" if logy else ""}</text>']
    if title:
        out.append(f'<text x="{width / 2}" y="28" text-anchor="middle" font-size="16">{title}</text>')
    for t in _ticks(x0, x1, logx):
        X = m + (t - x0) / (x1 - x0) * (width - 2 * m)
        lab = f"1e{int(t)}" if logx else f"{t:g}"
        out += [f'<line x1="{X:.1f}" y1="{height - m}" x2="{X:.1f}" y2="{height - m + 5}" stroke="black"/>',
                f'<line x1="{X:.1f}" y1="{m}" x2="{X:.1f}" y2="{height - m}" stroke="#dddddd"/>',
                f'<text x="{X:.1f}" y="{height - m + 20}" text-anchor="middle">{lab}</text>']
    for t in _ticks(y0, y1, logy):
        Y = height - m - (t - y0) / (y1 - y0) * (height - 2 * m)
        lab = f"1e{int(t)}" if logy else f"{t:g}"
        out += [f'<line x1="{m - 5}" y1="{Y:.1f}" x2="{m}" y2="{Y:.1f}" stroke="black"/>',
                f'<line x1="{m}" y1="{Y:.1f}" x2="{width - m}" y2="{Y:.1f}" stroke="#dddddd"/>',
                f'<text x="{m - 8}" y="{Y + 4:.1f}" text-anchor="end">{lab}</text>']
    for i, s in enumerate(series):
        c = s.get("color", COLORS[i % len(COLORS)])
        style = s.get("style", "both")
        if "curve_x" in s:
            pts = " ".join(f"{a:.1f},{b:.1f}" for a, b in zip(px(s["curve_x"]), py(s["curve_y"])) if np.isfinite(a + b))
            out.append(f'<polyline points="{pts}" fill="none" stroke="{c}" stroke-width="1.5" stroke-opacity="0.7"/>')
        X, Y = px(s["x"]), py(s["y"])
        if style in ("line", "both"):
            pts = " ".join(f"{a:.1f},{b:.1f}" for a, b in zip(X, Y) if np.isfinite(a + b))
            out.append(f'<polyline points="{pts}" fill="none" stroke="{c}" stroke-width="2"/>')
        if style in ("points", "both"):
            out += [f'<circle cx="{a:.1f}" cy="{b:.1f}" r="4" fill="{c}"/>' for a, b in zip(X, Y) if np.isfinite(a + b)]
        if s.get("star") is not None:
            a, b = float(px([s["star"][0]])[0]), float(py([s["star"][1]])[0])
            out.append(f'<path d="M {a:.1f} {b - 9:.1f} L {a + 7:.1f} {b + 7:.1f} L {a - 9:.1f} {b - 3:.1f} L {a + 9:.1f} {b - 3:.1f} '
                       f'L {a - 7:.1f} {b + 7:.1f} Z" fill="{c}" stroke="black"/>')
        out.append(f'<text x="{width - m - 250}" y="{m + 18 * i + 4}" fill="{c}">{s["name"]}</text>')
    out.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(out))


def write_table(path: Optional[str], header: Sequence[str], rows: Iterable[Sequence]) -> str:
    """CSV text of a table; written to ``path`` when given."""
    lines = [",".join(header)] + [",".join(f"{v:.6g}" if isinstance(v, float) else str(v) for v in r) for r in rows]
    text = "\n".join(lines) + "\n"
    if path:
        with open(path, "w") as f:
            f.write(text)
    return text
