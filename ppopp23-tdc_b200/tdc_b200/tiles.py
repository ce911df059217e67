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


def load_tables(paths=None):
    """{(C, N, H, W, B, R, stride): (Tile tuple, time_ms)} from the shipped (or given) CSVs."""
    out = {}
    for path in (paths if paths is not None else sorted(glob.glob(os.path.join(_TABLE_DIR, "*.csv")))):
        with open(path) as f:
            for row in csv.DictReader(f):
                if float(row["diff"]) != 0.0:
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
