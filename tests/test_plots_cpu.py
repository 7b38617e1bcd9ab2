"""Sweep analysis and figure writers: optima of synthetic sweeps, scaling exponents, subset sensitivity, file parsing, SVG output."""
import json
import xml.dom.minidom

import numpy as np
import pytest

from archscale_b200.plots import curves, hparam_sweeps as hs
from archscale_b200.plots.svg import line_chart


def _sweep_csv(tmp_path, law=lambda T: 3e-2 * (T / 1e9) ** -0.3):
    path = tmp_path / "runs.csv"
    rng = np.random.default_rng(0)
    lines = ["Name,metric/val_loss@1x"]
    for T in (1e9, 2e9, 4e9, 8e9, 16e9):
        best = law(T)
        for mult in (0.25, 0.5, 1.0, 2.0, 4.0):
            lr = best * mult
            loss = 2.0 + 0.1 * np.log(T / 1e9) * -1 + 0.05 * (np.log(lr) - np.log(best)) ** 2 + rng.normal(0, 1e-5)
            lines.append(f"scaling_mup_muonh_lr{lr:.6e}x_tok{T:.3e}_d16_ctx4096,{loss:.8f}")
    path.write_text("\n".join(lines) + "\n")
    return str(path)


def test_run_name_parsing():
    p = hs.parse_run_name("scaling_mup_muonh_lr4e-3x_tok1.04e10_bsz2e6_d16_ctx4096")
    assert p["lr"] == pytest.approx(4e-3) and p["tokens"] == pytest.approx(1.04e10) and p["bsz"] == 2e6 and p["depth"] == 16


def test_quadratic_optimum_and_scaling_exponent(tmp_path):
    recs = hs.load_runs(_sweep_csv(tmp_path))
    opt = hs.optima_by_group(recs, "tokens", "lr")
    assert len(opt) == 5
    for o in opt:
        assert o["opt_lr"] == pytest.approx(3e-2 * (o["tokens"] / 1e9) ** -0.3, rel=1e-3)
    p = hs.fit_power_law([o["tokens"] for o in opt], [o["opt_lr"] for o in opt])
    assert p[1] == pytest.approx(-0.3, abs=2e-3)
    loo = hs.leave_one_out([o["tokens"] for o in opt], [o["opt_lr"] for o in opt])
    assert len(loo) == 5 and all(abs(r["power_law_err_pct"]) < 1.0 for r in loo)
    assert np.isnan(hs.quadratic_optimum([1, 2, 4], [1.0, 2.0, 1.0])[0])           # a parabola that opens downwards has no optimum


def test_npoints_sensitivity_shrinks_with_more_points():
    rng = np.random.default_rng(1)
    lrs = np.geomspace(1e-3, 3e-2, 7)
    loss = 2.0 + 0.04 * (np.log(lrs) - np.log(6e-3)) ** 2 + rng.normal(0, 2e-3, 7)
    rows = hs.npoints_sensitivity(lrs, loss)
    assert [r["k"] for r in rows] == [3, 4, 5, 6]
    assert rows[-1]["opt_x_err_pct"] < rows[0]["opt_x_err_pct"]


def test_cli_writes_tables_and_well_formed_svg(tmp_path, capsys):
    path = _sweep_csv(tmp_path)
    for what in ("scaling", "npoints", "sweep"):
        svg = tmp_path / f"{what}.svg"
        assert hs.main([what, path, "--svg", str(svg)]) == 0
        xml.dom.minidom.parse(str(svg))
    out = capsys.readouterr().out
    assert "power_law" in out and "opt_lr" in out


def test_metric_curves_comparison_and_accuracy(tmp_path):
    m = tmp_path / "z.csv"
    m.write_text("Step,run_a_d8_x - attn_z_mean,run_a_d8_x - attn_z_mean__MIN,run_b_d16_x - attn_z_mean\n"
                 "10,1.0,0.5,2.0\n20,1.5,0.6,\n30,1.25,0.7,2.5\n")
    data = curves.load_metric(str(m), "attn_z_mean")
    assert list(data) == [8, 16] and data[8] == ([10.0, 20.0, 30.0], [1.0, 1.5, 1.25]) and data[16][0] == [10.0, 30.0]
    recs = [{"name": "muonh_d8", "depth": 8, "loss": 2.5}, {"name": "muonh_d8_b", "depth": 8, "loss": 2.4},
            {"name": "adamw_d8", "depth": 8, "loss": 2.6}, {"name": "muonh_d16", "depth": 16, "loss": 2.1}]
    cmp_ = curves.compare_variants(recs, "depth", ["muonh", "adamw"])
    assert cmp_["muonh"] == ([8, 16], [2.4, 2.1]) and cmp_["adamw"] == ([8], [2.6])
    d = tmp_path / "res"
    d.mkdir()
    (d / "mup_sambay_d16_swa512.json").write_text(json.dumps([{"mean_acc": 0.1, "std_acc": 0.0}, {"mean_acc": 0.8, "std_acc": 0.02}]))
    (d / "mup_sambay_d16_swa128.json").write_text(json.dumps([{"mean_acc": 0.6, "std_acc": 0.05}]))
    acc = curves.accuracy_by_window(str(d))
    assert acc == {"sambay": [(128, 0.6, 0.05), (512, 0.8, 0.02)]}
    svg = tmp_path / "acc.svg"
    assert curves.main(["accuracy", str(d), "--svg", str(svg), "--out", str(tmp_path / "acc.csv")]) == 0
    xml.dom.minidom.parse(str(svg))
    line_chart(str(svg), [{"name": "a", "x": [1, 2, 3], "y": [3.0, 2.0, 1.0]}], "x", "y")
    xml.dom.minidom.parse(str(svg))
