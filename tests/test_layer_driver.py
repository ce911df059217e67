"""The per-shape layer drivers (native and Python) and the table builder, run as a user would run them.

What the reference's generated drivers promise (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:
404-514): integer inputs 0..9 and all-ones weights give an L1 difference of exactly 0, and one CSV row per run in a
fixed column order.  The native driver reaches the library through its C ABI only."""
import csv
import os
import subprocess
import sys

import pytest

from helpers import ROOT

PKG = os.path.join(ROOT, "ppopp23-tdc_b200", "tdc_b200")
DRIVER = os.path.join(PKG, "layer_driver")


def test_native_driver_is_built_and_checks_its_arguments(built):
    assert os.path.exists(DRIVER), "python ppopp23-tdc_b200/build.py builds it"
    r = subprocess.run([DRIVER], capture_output=True, text=True)             # no shape: usage, before any CUDA call
    assert r.returncode == 2 and "usage" in r.stderr
    r = subprocess.run([DRIVER, "64", "64", "56", "56", "--tc", "2"], capture_output=True, text=True)
    assert r.returncode == 2


def _row(text):
    return [float(v) if v not in ("nan", "-nan") else float("nan") for v in text.strip().splitlines()[-1].split(",")]


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [("32", "32", "56", "56"), ("64", "64", "28", "28")])
def test_native_driver_rows(built, shape, tmp_path):
    out = tmp_path / "rows.csv"
    for extra, ncol in (([], 9), (["--tc", "4"], 9), (["--tc", "3", "--batch", "8"], 9), (["--reference-row"], 14),
                        (["--stride", "2", "--tc", "4"], 9), (["--filter", "1", "--pad", "0", "--batch", "3"], 9)):
        r = subprocess.run([DRIVER, *shape, "--iters", "5", "--csv", str(out)] + extra, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, (extra, r.stdout, r.stderr)
        row = _row(r.stdout)
        assert len(row) == ncol and row[-1] == 0.0, (extra, r.stdout)           # diff == 0: exact
        assert [int(v) for v in row[:4]] == [int(shape[1]), int(shape[0]), int(shape[2]), int(shape[3])]    # N,C,H,W
        if ncol == 14:
            assert row[8] > 0 and row[6] == row[6]      # TDC time; the implicit-GEMM class always runs
            assert abs(row[11] - row[6] / row[8]) <= 1e-3 * row[11]           # GEMM/TDC column
    rows = list(csv.reader(open(out)))
    assert len(rows) == 6 and [len(r) for r in rows] == [9, 9, 9, 14, 9, 9]


@pytest.mark.gpu
def test_python_driver_rows(built, tmp_path, capsys):
    from tdc_b200 import layer_driver
    out = tmp_path / "rows.csv"
    for argv, ncol in ((["--shape", "32,32,56,56", "--iters", "3"], 11), (["--shape", "64,64,28,28", "--tc", "3", "--iters", "3"], 11),
                       (["--shape", "64,64,28,28", "--tc", "4", "--iters", "3", "--batch", "4"], 11),
                       (["--shape", "32,32,56,56", "--reference-row", "--iters", "3"], 14)):
        assert layer_driver.main(argv + ["--csv", str(out)]) == 0
        row = capsys.readouterr().out.strip().splitlines()[-1].split(",")
        assert len(row) == ncol and float(row[-1]) == 0.0
    assert [len(r) for r in csv.reader(open(out))] == [11, 11, 11, 14]


@pytest.mark.gpu
def test_table_builder_on_a_small_shape_list(built, tmp_path):
    from tdc_b200 import tune
    table, best = tmp_path / "table.csv", tmp_path / "best.csv"
    tune.main(["--batch", "2", "--shape-list", "8,16,8,8,3,1,1;16,8,7,7,1,1,0", "--max-per-shape", "6", "--model-top", "3",
               "--iters", "1", "--out", str(table), "--best-out", str(best)])
    rows = list(csv.DictReader(open(table)))
    assert rows and list(rows[0].keys()) == tune.COLUMNS
    assert all(float(r["diff"]) == 0.0 and float(r["time_ms"]) > 0 for r in rows)
    assert {(int(r["C"]), int(r["N"])) for r in rows} == {(8, 16), (16, 8)}
    assert len(list(csv.DictReader(open(best)))) == 2
    # the reference's tables are read from both ends: the first seven and the last three of its ten columns
    assert tune.COLUMNS[:10] == ["C", "N", "H", "W", "th", "tw", "tc", "occupancy", "diff", "time_ms"]
