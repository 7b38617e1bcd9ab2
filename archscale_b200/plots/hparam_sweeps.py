"""Hyper-parameter sweep analysis: optimal learning rate / batch size per budget, their scaling with the token budget, and how
many sweep points the optimum needs.

Behavioural reference (the arithmetic of the reference's figure scripts, which read an experiment-tracker export with one row
per run and the hyper-parameters encoded in the run name):

* per budget, a parabola in log(lr) through (lr, validation loss) gives the optimal lr and loss
  (`plots/plot_lr_scaling.py:40-66`, `plots/plot_optimal_hparams.py:65-80`, `plots/plot_combined_lr_sweep.py`);
* the optima follow ``a·T^b`` or ``a·T^b + c`` in the token budget T; leave-one-out extrapolation compares the two
  (`plots/plot_lr_scaling.py:83-96,187-247`; the same with batch size in `plots/plot_bsz_scaling.py`);
* the mean relative error of the optimum fitted from every k-subset of a sweep's points against the fit through all of them
  (`plots/plot_npoints_relative_error.py:43-92`, `plots/plot_lr_npoints_sensitivity.py`, `plots/plot_loss_npoints_sensitivity.py`).

    python -m archscale_b200.plots.hparam_sweeps scaling runs.csv --x lr --metric "metric/val_loss@1x" --svg lr_scaling.svg
    python -m archscale_b200.plots.hparam_sweeps scaling runs.csv --x bsz
    python -m archscale_b200.plots.hparam_sweeps npoints runs.csv --svg npoints.svg
    python -m archscale_b200.plots.hparam_sweeps sweep runs.csv --group depth --svg sweep.svg
"""
from __future__ import annotations

import argparse
import csv
import re
import sys
from itertools import combinations
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .svg import line_chart, write_table

_PATTERNS = {"lr": r"_lr([\d.e\-]+)x?", "tokens": r"_tok([\d.e+]+)", "bsz": r"_bsz([\d.e+]+)", "depth": r"_d(\d+)(?:_|$)",
             "wd": r"_wd([\d.e\-]+)", "top_k": r"_k(\d+)(?:_|$)", "sparsity": r"_s(\d+)(?:_|$)"}


def parse_run_name(name: str) -> Dict[str, float]:
    """Hyper-parameters encoded in a run name (``…_lr4e-3x_tok1.04e10_bsz2e6_d16_…``); absent ones are left out."""
    out: Dict[str, float] = {}
    for key, pat in _PATTERNS.items():
        m = re.search(pat, name)
        if m:
            try:
                out[key] = float(m.group(1).rstrip("."))
            except ValueError:
                pass
    return out


def load_runs(path: str, metric: str = "metric/val_loss@1x", name_col: str = "Name") -> List[Dict[str, float]]:
    """Rows of a tracker export → records with the parsed hyper-parameters and ``loss``."""
    rows = []
    with open(path, newline="") as f:
        for r in csv.DictReader(f):
            if not r.get(metric):
                continue
            rec = parse_run_name(r[name_col])
            rec["loss"] = float(r[metric])
            rec["name"] = r[name_col]
            rows.append(rec)
    return rows


def quadratic_optimum(x: Sequence[float], loss: Sequence[float]) -> Tuple[float, float, np.ndarray]:
    """Parabola in log(x) through the points → (optimal x, loss there, coefficients); NaNs when it opens downwards."""
    lx = np.log(np.asarray(x, dtype=np.float64))
    c = np.polyfit(lx, np.asarray(loss, dtype=np.float64), 2)
    if c[0] <= 0:
        return float("nan"), float("nan"), c
    opt = -c[1] / (2 * c[0])
    return float(np.exp(opt)), float(np.polyval(c, opt)), c


def optima_by_group(records: Iterable[Dict[str, float]], group: str, x: str) -> List[Dict[str, float]]:
    groups: Dict[float, List[Dict[str, float]]] = {}
    for r in records:
        if group in r and x in r:
            groups.setdefault(r[group], []).append(r)
    out = []
    for g in sorted(groups):
        pts = sorted(groups[g], key=lambda r: r[x])
        if len(pts) < 3:
            continue
        ox, ol, c = quadratic_optimum([p[x] for p in pts], [p["loss"] for p in pts])
        out.append({group: g, "opt_" + x: ox, "opt_loss": ol, "n": len(pts), "coeffs": c,
                    "xs": [p[x] for p in pts], "losses": [p["loss"] for p in pts]})
    return out


def power_law(T, a, b):
    return a * np.power(T, b)


def power_law_irr(T, a, b, c):
    return a * np.power(T, b) + c


def fit_power_law(T: Sequence[float], y: Sequence[float], irreducible: bool = False) -> np.ndarray:
    """Least squares of ``a·T^b`` (or ``a·T^b + c``).  T is divided by its geometric mean for the solver and the returned ``a``
    refers to the unscaled T."""
    from scipy.optimize import curve_fit
    T, y = np.asarray(T, dtype=np.float64), np.asarray(y, dtype=np.float64)
    s = float(np.exp(np.mean(np.log(T))))
    b0 = np.polyfit(np.log(T / s), np.log(np.abs(y) + 1e-300), 1)
    if irreducible:
        p, _ = curve_fit(power_law_irr, T / s, y, p0=[float(np.exp(b0[1])), float(b0[0]), 0.0], maxfev=20000)
        return np.array([p[0] * s ** (-p[1]), p[1], p[2]])
    p, _ = curve_fit(power_law, T / s, y, p0=[float(np.exp(b0[1])), float(b0[0])], maxfev=20000)
    return np.array([p[0] * s ** (-p[1]), p[1]])


def leave_one_out(T: Sequence[float], y: Sequence[float]) -> List[Dict[str, float]]:
    """Fit both laws without point i and predict it: one row per held-out point with the signed relative errors in percent."""
    T, y = np.asarray(T, dtype=np.float64), np.asarray(y, dtype=np.float64)
    rows = []
    for i in range(len(T)):
        keep = np.arange(len(T)) != i
        row = {"held_out": float(T[i]), "true": float(y[i])}
        for key, irr, fn in (("power_law", False, power_law), ("power_law_irr", True, power_law_irr)):
            try:
                if irr and keep.sum() < 4:
                    raise RuntimeError("three parameters need four points")
                p = fit_power_law(T[keep], y[keep], irreducible=irr)
                pred = float(fn(T[i], *p))
            except (RuntimeError, ValueError):
                pred = float("nan")
            row[key] = pred
            row[key + "_err_pct"] = (pred - y[i]) / y[i] * 100
        rows.append(row)
    return rows


def npoints_sensitivity(x: Sequence[float], loss: Sequence[float]) -> List[Dict[str, float]]:
    """For k = 3 … n−1: mean relative error (percent) of the optimum fitted from every k-subset against the fit through all n."""
    x, loss = np.asarray(x, dtype=np.float64), np.asarray(loss, dtype=np.float64)
    n = len(x)
    full_x, full_loss, _ = quadratic_optimum(x, loss)
    rows = []
    for k in range(3, n):
        ex, el = [], []
        for combo in combinations(range(n), k):
            idx = list(combo)
            ox, ol, _ = quadratic_optimum(x[idx], loss[idx])
            if np.isfinite(ox):
                ex.append(abs(ox - full_x) / full_x)
                el.append(abs(ol - full_loss) / full_loss)
        rows.append({"k": k, "opt_x_err_pct": float(np.mean(ex) * 100) if ex else float("nan"),
                     "opt_loss_err_pct": float(np.mean(el) * 100) if el else float("nan"), "subsets": len(ex)})
    return rows


def _sweep_series(opt: List[Dict], group: str, x: str) -> List[Dict]:
    series = []
    for o in opt:
        lx = np.linspace(np.log(min(o["xs"])) - 0.3, np.log(max(o["xs"])) + 0.3, 100)
        s = {"name": f"{group} {o[group]:g}: best {x} {o['opt_' + x]:.4g}, loss {o['opt_loss']:.4f}", "x": o["xs"],
             "y": o["losses"], "style": "points", "curve_x": np.exp(lx), "curve_y": np.polyval(o["coeffs"], lx)}
        if np.isfinite(o["opt_" + x]):
            s["star"] = (o["opt_" + x], o["opt_loss"])
        series.append(s)
    return series


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=("scaling", "npoints", "sweep"))
    ap.add_argument("path")
    ap.add_argument("--metric", default="metric/val_loss@1x")
    ap.add_argument("--name-col", default="Name")
    ap.add_argument("--x", default="lr", help="swept hyper-parameter (lr, bsz, wd)")
    ap.add_argument("--group", default="tokens", help="one sweep per value of this key (tokens, depth, …)")
    ap.add_argument("--svg", default=None)
    ap.add_argument("--out", default=None, help="CSV of the table (default: stdout)")
    a = ap.parse_args(argv)
    recs = load_runs(a.path, a.metric, a.name_col)
    opt = optima_by_group(recs, a.group, a.x)
    if not opt:
        print(f"no group of {a.group!r} has three runs with {a.x!r} in its name", file=sys.stderr)
        return 1
    if a.what == "sweep":
        text = write_table(a.out, [a.group, "opt_" + a.x, "opt_loss", "n"], [[o[a.group], o["opt_" + a.x], o["opt_loss"], o["n"]] for o in opt])
        if a.svg:
            line_chart(a.svg, _sweep_series(opt, a.group, a.x), a.x, "validation loss", logx=True)
    elif a.what == "scaling":
        good = [o for o in opt if np.isfinite(o["opt_" + a.x])]
        T, y = [o[a.group] for o in good], [o["opt_" + a.x] for o in good]
        p = fit_power_law(T, y)
        rows = [["power_law", p[0], p[1], 0.0]]
        p3 = None
        if len(T) >= 4:
            p3 = fit_power_law(T, y, irreducible=True)
            rows.append(["power_law_irr", p3[0], p3[1], p3[2]])
        text = write_table(a.out, ["law", "a", "b", "c"], rows)
        text += write_table(None, ["held_out", "true", "power_law", "power_law_err_pct", "power_law_irr", "power_law_irr_err_pct"],
                            [[r["held_out"], r["true"], r["power_law"], r["power_law_err_pct"], r["power_law_irr"], r["power_law_irr_err_pct"]]
                             for r in leave_one_out(T, y)])
        if a.svg:
            grid = np.geomspace(min(T) * 0.5, max(T) * 3, 100)
            series = [{"name": f"optimal {a.x}: {p[0]:.3g}·T^{p[1]:.3f}", "x": T, "y": y, "style": "points",
                       "curve_x": grid, "curve_y": power_law(grid, *p)}]
            if p3 is not None:
                series.append({"name": f"with offset {p3[2]:.3g}", "x": T, "y": y, "style": "points", "curve_x": grid,
                               "curve_y": power_law_irr(grid, *p3)})
            line_chart(a.svg, series, a.group, "optimal " + a.x, logx=True, logy=True)
    else:
        rows, series = [], []
        for o in opt:
            sens = npoints_sensitivity(o["xs"], o["losses"])
            rows += [[o[a.group], s["k"], s["opt_x_err_pct"], s["opt_loss_err_pct"], s["subsets"]] for s in sens]
            if sens:
                series.append({"name": f"{a.group} {o[a.group]:g}", "x": [s["k"] for s in sens],
                               "y": [max(s["opt_x_err_pct"], 1e-6) for s in sens]})
        text = write_table(a.out, [a.group, "k", "opt_" + a.x + "_err_pct", "opt_loss_err_pct", "subsets"], rows)
        if a.svg and series:
            line_chart(a.svg, series, "sweep points used", f"mean relative error of the optimal {a.x} (%)", logy=True)
    if not a.out:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
