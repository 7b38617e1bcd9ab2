"""Scaling-law fits of validation loss against training FLOPs or tokens.

Behavioural reference: `plot_flops_scaling.py:19-60,98-140` and `plot_data_scaling.py` of the reference fit
``L = A · X^(−b) + C`` per model family (X = FLOPs from the depth law ``N = mult·d³``, ``T = t0·N/N0``, ``C = 6·N·T``,
or X = training tokens) with ``scipy.optimize.curve_fit`` and draw the curves with matplotlib.  This module does the
fitting and the table; it writes CSV (and a dependency-free SVG) instead of needing a plotting library.

    python -m archscale_b200.plots.scaling_fit flops            # published depth sweep (d8…d24), fitted exponents
    python -m archscale_b200.plots.scaling_fit data --svg out.svg
    python -m archscale_b200.plots.scaling_fit csv runs.csv --x flops --y val_loss --group model
"""
from __future__ import annotations

import argparse
import csv
import sys
from typing import Dict, Iterable, List, Sequence, Tuple

import numpy as np

# validation losses published in the reference's plot scripts (`plot_flops_scaling.py:20-25`, `plot_data_scaling.py:22-25`)
DEPTHS = (8, 12, 16, 20, 24)
FLOPS_SWEEP: Dict[str, Tuple[float, ...]] = {
    "Transformer++ (SP)": (2.6746, 2.2836, 2.0831, 1.9454, 1.8360),
    "Transformer++ (muP)": (2.5972, 2.2647, 2.0682, 1.9263, 1.8252),
    "Transformer++ (muP++)": (2.5621, 2.2440, 2.0505, 1.9164, 1.8172),
    "Samba+YOCO (muP++)": (2.5014, 2.2040, 2.0213, 1.8957, 1.79928),
    "SambaY (muP++)": (2.5051, 2.2073, 2.0227, 1.8963, 1.7999),
}
TOKENS_B = (100, 200, 300, 400, 500, 600)
DATA_SWEEP: Dict[str, Tuple[float, ...]] = {
    "Transformer++ (SP)": (2.0707, 2.0128, 1.9908, 1.9753, 1.9637, 1.9541),
    "Transformer++ (muP++, batch scaling)": (2.0516, 2.0027, 1.9784, 1.9656, 1.9535, 1.9461),
    "SambaY (muP++)": (2.0242, 1.9766, 1.9548, 1.9385, 1.9311, 1.92245),
    "Samba+YOCO (muP++)": (2.0212, 1.9736, 1.9509, 1.9377, 1.9272, 1.9209),
}


def depth_to_flops(depth: float, ar: int = 128, base_depth: int = 16, base_tokens: float = 1e11, mult: float = 14.5) -> float:
    """FLOPs of the depth-``d`` run of the sweep: ``N = mult·ar²·d³``, tokens scale with N from ``base_tokens`` at
    ``base_depth``, ``C = 6·N·T`` (`plot_flops_scaling.py:27-46`)."""
    n = mult * ar ** 2 * depth ** 3
    n0 = mult * ar ** 2 * base_depth ** 3
    return 6.0 * n * (base_tokens * n / n0)


def power_law_with_offset(x, A, b, C):
    return A * np.power(x, -b) + C


def fit_power_law(x: Sequence[float], y: Sequence[float]) -> Dict[str, float]:
    """Least-squares fit of ``y = A·x^(−b) + C``; x is rescaled by its geometric mean for conditioning and the returned
    ``A`` refers to the unscaled x.  Returns A, b, C and the root-mean-square residual."""
    from scipy.optimize import curve_fit
    x, y = np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64)
    s = float(np.exp(np.mean(np.log(x))))
    xs = x / s
    p0 = (max(y[0] - y[-1], 1e-3), 0.3, max(y.min() - 0.1, 0.0))
    popt, _ = curve_fit(power_law_with_offset, xs, y, p0=p0, maxfev=20000,
                        bounds=((0.0, 0.0, 0.0), (np.inf, 5.0, float(y.min()))))
    A, b, C = (float(v) for v in popt)
    rms = float(np.sqrt(np.mean((power_law_with_offset(xs, A, b, C) - y) ** 2)))
    return {"A": A * s ** b, "b": b, "C": C, "rms": rms}


def fit_families(x: Sequence[float], families: Dict[str, Sequence[float]]) -> List[Dict]:
    rows = []
    for name, losses in families.items():
        f = fit_power_law(x, losses)
        rows.append({"family": name, **f})
    return rows


def read_csv(path: str, x: str, y: str, group: str) -> Dict[str, Tuple[List[float], List[float]]]:
    """Rows of a metrics export → {group: (xs, ys)} sorted by x."""
    out: Dict[str, Tuple[List[float], List[float]]] = {}
    with open(path, newline="") as f:
        for row in csv.DictReader(f):
            if row.get(x) in (None, "") or row.get(y) in (None, ""):
                continue
            xs, ys = out.setdefault(row.get(group, "all") or "all", ([], []))
            xs.append(float(row[x]))
            ys.append(float(row[y]))
    for k, (xs, ys) in out.items():
        order = np.argsort(xs)
        out[k] = ([xs[i] for i in order], [ys[i] for i in order])
    return out


def write_svg(path: str, series: Iterable[Tuple[str, Sequence[float], Sequence[float], Dict[str, float]]],
              xlabel: str, ylabel: str = "validation loss") -> None:
    """Log-x plot of the points and fitted curves as a plain SVG file."""
    series = list(series)
    W, H, m = 900, 600, 70
    allx = np.concatenate([np.asarray(s[1], dtype=np.float64) for s in series])
    ally = np.concatenate([np.asarray(s[2], dtype=np.float64) for s in series])
    lx0, lx1 = np.log10(allx.min()) - 0.05, np.log10(allx.max()) + 0.05
    y0, y1 = ally.min() - 0.03, ally.max() + 0.03
    px = lambda v: m + (np.log10(v) - lx0) / (lx1 - lx0) * (W - 2 * m)
    py = lambda v: H - m - (v - y0) / (y1 - y0) * (H - 2 * m)
    colors = ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b"]
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="13">',
             f'<rect width="{W}" height="{H}" fill="white"/>',
             f'<line x1="{m}" y1="{H - m}" x2="{W - m}" y2="{H - m}" stroke="black"/>',
             f'<line x1="{m}" y1="{m}" x2="{m}" y2="{H - m}" stroke="black"/>',
             f'<text x="{W / 2}" y="{H - 20}" text-anchor="middle">{xlabel} (log scale)</text>',
             f'<text x="20" y="{H / 2}" text-anchor="middle" transform="rotate(-90 20 {H / 2})">{ylabel}</text>']
    for i, (name, xs, ys, fit) in enumerate(series):
        c = colors[i % len(colors)]
        grid = np.logspace(np.log10(min(xs)), np.log10(max(xs)), 60)
        pts = " ".join(f"{px(g):.1f},{py(power_law_with_offset(g, fit['A'], fit['b'], fit['C'])):.1f}" for g in grid)
        parts.append(f'<polyline points="{pts}" fill="none" stroke="{c}" stroke-width="2"/>')
        parts += [f'<circle cx="{px(a):.1f}" cy="{py(b):.1f}" r="4" fill="{c}"/>' for a, b in zip(xs, ys)]
        parts.append(f'<text x="{W - m - 330}" y="{m + 18 * i}" fill="{c}">{name}: b={fit["b"]:.3f}, C={fit["C"]:.3f}</text>')
    parts.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(parts))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=("flops", "data", "csv"))
    ap.add_argument("path", nargs="?")
    ap.add_argument("--x", default="flops")
    ap.add_argument("--y", default="val_loss")
    ap.add_argument("--group", default="model")
    ap.add_argument("--svg", default=None)
    ap.add_argument("--out", default=None, help="CSV file for the fitted parameters (default: stdout)")
    a = ap.parse_args(argv)
    if a.what == "flops":
        xs = [depth_to_flops(d) for d in DEPTHS]
        groups = {k: (xs, list(v)) for k, v in FLOPS_SWEEP.items()}
        xlabel = "training FLOPs"
    elif a.what == "data":
        xs = [t * 1e9 for t in TOKENS_B]
        groups = {k: (xs, list(v)) for k, v in DATA_SWEEP.items()}
        xlabel = "training tokens"
    else:
        if not a.path:
            ap.error("csv needs a path")
        groups = read_csv(a.path, a.x, a.y, a.group)
        xlabel = a.x
    rows, series = [], []
    for name, (gx, gy) in groups.items():
        if len(gx) < 3:
            continue
        fit = fit_power_law(gx, gy)
        rows.append({"family": name, **fit})
        series.append((name, gx, gy, fit))
    w = csv.DictWriter(open(a.out, "w", newline="") if a.out else sys.stdout, fieldnames=["family", "A", "b", "C", "rms"])
    w.writeheader()
    for r in rows:
        w.writerow({k: (f"{v:.6g}" if isinstance(v, float) else v) for k, v in r.items()})
    if a.svg and series:
        write_svg(a.svg, series, xlabel)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
