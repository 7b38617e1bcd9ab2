"""Training-curve and comparison figures from tracker exports and evaluation result files.

Behavioural reference:

* stability metrics over training per depth — columns ``"<run name> - <metric>"`` of a tracker CSV with a ``Step`` column, the
  ``__MIN`` / ``__MAX`` companions dropped, the run's depth read from ``_d<depth>_`` in its name, steps converted to tokens
  (`plots/plot_stability.py:39-86`, `plots/plot_ablation_stability.py`);
* final-loss comparisons between variants of one sweep (`plots/plot_muonh_comparison.py`, `plots/plot_qknorm_comparison.py`,
  `plots/plot_scaling_comparison.py`, `plots/plot_moe_ablation.py`, `plots/plot_moe_k_scaling.py`, `plots/plot_moe_s_scaling.py`,
  `plots/plot_balloss.py`): one line per variant over the swept quantity;
* long-context accuracy against the sliding-window size — one JSON file per (model, window) whose last entry holds ``mean_acc`` /
  ``std_acc``, the model and window read from the file name (`plots/plot_accuracy.py:18-75`).

    python -m archscale_b200.plots.curves metric stability/attn_z_mean.csv --metric attn_z_mean --tokens-per-step 1.0e7 --svg z.svg
    python -m archscale_b200.plots.curves compare runs.csv --x depth --variant "muonh|muon|adamw" --svg cmp.svg
    python -m archscale_b200.plots.curves accuracy prolong_results_32k --svg acc.svg
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
import sys
from typing import Dict, List, Optional, Sequence, Tuple

from .hparam_sweeps import load_runs
from .svg import line_chart, write_table


def extract_depth(column: str) -> Optional[int]:
    m = re.search(r"_d(\d+)_", column)
    return int(m.group(1)) if m else None


def load_metric(path: str, metric: str) -> Dict[int, Tuple[List[float], List[float]]]:
    """{depth: (steps, values)} for the columns of ``path`` that carry ``metric`` (mean columns only), sorted by step."""
    with open(path, newline="") as f:
        rows = list(csv.DictReader(f))
    if not rows:
        return {}
    cols = [c for c in rows[0] if metric in c and "__MIN" not in c and "__MAX" not in c and extract_depth(c) is not None]
    out: Dict[int, Tuple[List[float], List[float]]] = {}
    for c in cols:
        d = extract_depth(c)
        if d in out:
            continue
        pts = sorted((float(r["Step"]), float(r[c])) for r in rows if r.get(c) not in (None, ""))
        out[d] = ([p[0] for p in pts], [p[1] for p in pts])
    return dict(sorted(out.items()))


def compare_variants(records: List[Dict], x: str, variants: Sequence[str]) -> Dict[str, Tuple[List[float], List[float]]]:
    """Best loss per value of ``x`` for every variant (a variant = a substring of the run name)."""
    out: Dict[str, Tuple[List[float], List[float]]] = {}
    for v in variants:
        best: Dict[float, float] = {}
        for r in records:
            if v in r["name"] and x in r:
                best[r[x]] = min(best.get(r[x], float("inf")), r["loss"])
        if best:
            xs = sorted(best)
            out[v] = (xs, [best[k] for k in xs])
    return out


def accuracy_by_window(results_dir: str, model_pattern: str = r"mup_(.+?)_d\d+") -> Dict[str, List[Tuple[int, float, float]]]:
    """{model: [(window, mean_acc, std_acc), …]} from the JSON files of ``results_dir``; files without ``swa<N>`` count as
    window 0 (full attention)."""
    out: Dict[str, List[Tuple[int, float, float]]] = {}
    for fn in sorted(os.listdir(results_dir)):
        if not fn.endswith(".json"):
            continue
        m = re.search(model_pattern, fn)
        if not m:
            continue
        w = re.search(r"swa(\d+)", fn)
        with open(os.path.join(results_dir, fn)) as f:
            data = json.load(f)
        if not data:
            continue
        last = data[-1]
        out.setdefault(m.group(1), []).append((int(w.group(1)) if w else 0, float(last["mean_acc"]), float(last.get("std_acc", 0.0))))
    for k in out:
        out[k].sort()
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=("metric", "compare", "accuracy"))
    ap.add_argument("path")
    ap.add_argument("--metric", default="metric/val_loss@1x")
    ap.add_argument("--tokens-per-step", type=float, default=None)
    ap.add_argument("--x", default="depth")
    ap.add_argument("--variant", default="", help="'|'-separated substrings of the run names to compare")
    ap.add_argument("--svg", default=None)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    if a.what == "metric":
        data = load_metric(a.path, a.metric)
        k = (a.tokens_per_step or 1.0) / (1e9 if a.tokens_per_step else 1.0)
        rows = [[d, s * k, v] for d, (st, va) in data.items() for s, v in zip(st, va)]
        text = write_table(a.out, ["depth", "tokens_B" if a.tokens_per_step else "step", a.metric], rows)
        if a.svg:
            line_chart(a.svg, [{"name": f"d{d}", "x": [s * k for s in st], "y": va, "style": "line"} for d, (st, va) in data.items()],
                       "training tokens (B)" if a.tokens_per_step else "step", a.metric)
    elif a.what == "compare":
        recs = load_runs(a.path, a.metric)
        cmp_ = compare_variants(recs, a.x, [v for v in a.variant.split("|") if v])
        text = write_table(a.out, ["variant", a.x, "loss"], [[v, x, y] for v, (xs, ys) in cmp_.items() for x, y in zip(xs, ys)])
        if a.svg:
            line_chart(a.svg, [{"name": v, "x": xs, "y": ys} for v, (xs, ys) in cmp_.items()], a.x, "validation loss")
    else:
        acc = accuracy_by_window(a.path)
        text = write_table(a.out, ["model", "window", "mean_acc", "std_acc"], [[m, w, mu, sd] for m, pts in acc.items() for w, mu, sd in pts])
        if a.svg:
            line_chart(a.svg, [{"name": m, "x": [max(p[0], 1) for p in pts], "y": [p[1] for p in pts]} for m, pts in acc.items()],
                       "sliding-window size", "accuracy", logx=True)
    if not a.out:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
