"""Scaling-law fitting utility: recovers a known power law, fits the published sweeps, reads a CSV export (CPU)."""
import csv

import numpy as np

from archscale_b200.plots import scaling_fit as sf


def test_fit_recovers_known_law():
    x = np.logspace(18, 22, 8)
    y = 300.0 * x ** -0.12 + 1.5
    f = sf.fit_power_law(x, y)
    assert abs(f["b"] - 0.12) < 5e-3 and abs(f["C"] - 1.5) < 2e-2 and f["rms"] < 1e-4


def test_published_sweeps_fit_and_flops_law():
    assert abs(sf.depth_to_flops(16) - 6 * (14.5 * 128 ** 2 * 16 ** 3) * 1e11) / sf.depth_to_flops(16) < 1e-12
    xs = [sf.depth_to_flops(d) for d in sf.DEPTHS]
    rows = sf.fit_families(xs, sf.FLOPS_SWEEP)
    assert len(rows) == 5 and all(r["rms"] < 1e-2 and 0.0 < r["b"] < 1.0 for r in rows)
    # the muP++ runs reach a lower loss than standard parametrisation at every depth of the sweep
    assert all(a < b for a, b in zip(sf.FLOPS_SWEEP["Transformer++ (muP++)"], sf.FLOPS_SWEEP["Transformer++ (SP)"]))


def test_csv_roundtrip_and_svg(tmp_path):
    p = tmp_path / "runs.csv"
    with open(p, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["model", "flops", "val_loss"])
        for name, off in (("a", 1.0), ("b", 1.2)):
            for x in (1e19, 3e19, 1e20, 3e20, 1e21):
                w.writerow([name, x, 100.0 * x ** -0.1 + off])
    groups = sf.read_csv(str(p), "flops", "val_loss", "model")
    assert set(groups) == {"a", "b"} and len(groups["a"][0]) == 5
    out, svg = tmp_path / "fit.csv", tmp_path / "fit.svg"
    assert sf.main(["csv", str(p), "--out", str(out), "--svg", str(svg)]) == 0
    rows = list(csv.DictReader(open(out)))
    assert {r["family"] for r in rows} == {"a", "b"} and all(abs(float(r["b"]) - 0.1) < 1e-2 for r in rows)
    assert svg.read_text().startswith("<svg")
