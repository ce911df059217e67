"""Tile choice the way the reference makes it: a measured table first, the model second.

The reference ships one measured table per GPU and picks the fastest row per shape for its
ORACLE kernels (A100-evaluation/TDC-LAYERS-ORACLE/gen_from_occupancy.py:51-66,159-169), and
an analytical choice for its MODELING kernels (A100-evaluation/TDC-LAYERS-MODELING/model.py).
`best_tile` does the same for B200: rows of tables/*.csv (written by tdc_b200.tune on a B200;
same ten leading columns as the reference tables) are looked up by shape and batch; a shape
that is not in a table gets the analytical choice of tdc_select_tile.
"""
import csv
import glob
import os

from . import ops
from ._lib import Tile

_TABLE_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tables")
_FIELDS = ("th", "tw", "tc", "tn", "nog", "gy", "gx", "imgs", "ks")
_table = None


REFERENCE_COLUMNS = ("C", "N", "H", "W", "th", "tw", "tc", "occupancy", "diff", "time_ms")


def read_rows(path):
    """Rows of a table as dicts.  Tables written by tdc_b200.tune start with a header line; the
    reference's own tables (a100-occupancy-unrolled, 2080Ti-occupancy*) have none and hold
    exactly the ten REFERENCE_COLUMNS — both load."""
    with open(path) as f:
        first = f.readline()
        f.seek(0)
        if first.split(",")[0].strip().isdigit():
            return [dict(zip(REFERENCE_COLUMNS, (v.strip() for v in ln.split(",")))) for ln in f if ln.strip()]
        return list(csv.DictReader(f))


def query_best(rows, C, N, H, W, B=None):
    """Fastest row of a shape (the reference's query_best,
    A100-evaluation/TDC-LAYERS-ORACLE/gen_from_occupancy.py:51-66), exact match on the shape
    columns; `B` filters tables that have a batch column."""
    best = None
    for r in rows:
        if (int(r["C"]), int(r["N"]), int(r["H"]), int(r["W"])) != (C, N, H, W):
            continue
        if B is not None and "B" in r and int(r["B"]) != B:
            continue
        if best is None or float(r["time_ms"]) < float(best["time_ms"]):
            best = r
    return best


def load_tables(paths=None):
    """{(C, N, H, W, B, R, stride): (Tile tuple, time_ms)} from the shipped (or given) CSVs."""
    out = {}
    for path in (paths if paths is not None else sorted(glob.glob(os.path.join(_TABLE_DIR, "*.csv")))):
        for row in read_rows(path):
            if True:
                if float(row["diff"]) != 0.0 or "tn" not in row:     # reference tables carry no B200 tile fields
                    continue
                key = tuple(int(row[k]) for k in ("C", "N", "H", "W", "B")) + (int(row.get("R", 3) or 3),
                                                                              int(row.get("stride", 1) or 1))
                t = float(row["time_ms"])
                if key not in out or t < out[key][1]:
                    out[key] = (tuple(int(row[k]) for k in _FIELDS) + (int(row.get("kc", 1) or 1),), t)
    return out


def table_tile(B, C, H, W, K, R=3, S=3, pad=1, stride=1):
    """The measured-table pick, or None."""
    global _table
    if _table is None:
        _table = load_tables()
    if R != S or pad != (R - 1) // 2:
        return None
    hit = _table.get((C, K, H, W, B, R, stride))
    return Tile(*hit[0]) if hit else None


def best_tile(B, C, H, W, K, R=3, S=3, pad=1, stride=1, dev=None):
    t = table_tile(B, C, H, W, K, R, S, pad, stride)
    return t if t is not None else ops.select_tile(B, C, H, W, K, R, S, pad, stride, dev=dev)
