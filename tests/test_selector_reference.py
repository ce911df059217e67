"""The reference's tile selectors: the CPU restatement (oracle/selector_ref.py) against picks
made by the reference's own functions (tests/golden/selector_picks.json), and the table
reader against the reference's table format."""
import json
import os

import pytest

import ref_import
import selector_ref as S
from helpers import GOLDEN

PICKS = json.load(open(os.path.join(GOLDEN, "selector_picks.json")))
TABLES = {"A100": ("A100-evaluation/TDC-LAYERS-MODELING/a100-occupancy-unrolled", S.A100),
          "2080Ti": ("2080Ti-evaluation/TDC-LAYERS-MODELING/2080Ti-occupancy-unrolled", S.TI2080)}


def test_golden_holds_the_published_known_answers():
    a = PICKS["A100"]["shapes"]
    assert a["32,32,56,56"]["model"] == [1, 2, 16] and a["32,32,56,56"]["best"] == [2, 6, 16]
    assert abs(a["32,32,56,56"]["best_ms"] - 0.02573) < 5e-6 and abs(a["64,64,56,56"]["best_ms"] - 0.05485) < 5e-6
    t = PICKS["2080Ti"]["shapes"]
    assert t["32,32,56,56"]["best"] == [1, 4, 32] and t["192,160,7,7"]["model"] == [1, 2, 16]
    assert abs(PICKS["A100"]["mean_loss"] - 0.149) < 1e-3 and abs(PICKS["2080Ti"]["mean_loss"] - 0.239) < 1e-3
    assert all(v["model"][0] == 1 for v in a.values())           # the slice-before-sort quirk: th = 1 on A100


@pytest.mark.parametrize("gpu", ["A100", "2080Ti"])
def test_restatement_reproduces_every_pick(gpu):
    rel, consts = TABLES[gpu]
    path = os.path.join(ref_import.REFERENCE_ROOT, rel)
    if not os.path.isfile(path):
        pytest.skip("reference tables are not mounted")
    lines = S.read_lines(path)
    assert len(lines) == PICKS[gpu]["rows"]
    out, mean = S.replay(lines, consts)
    for shape, got in out.items():
        want = PICKS[gpu]["shapes"]["%d,%d,%d,%d" % shape]
        assert list(got["model"]) == want["model"], shape
        assert list(got["best"]) == want["best"], shape
        assert got["model_ms"] == want["model_ms"] and got["best_ms"] == want["best_ms"]
    assert abs(mean - PICKS[gpu]["mean_loss"]) < 1e-12


def test_table_reader_takes_the_reference_format(built, tmp_path):
    from tdc_b200 import tiles
    ref = tmp_path / "ref-occupancy"
    ref.write_text("64,32,224,224,1,7,1,0.5,0,2.14598\n64,32,224,224,1,7,2,0.5,0,1.1615\n32,32,56,56,2,6,16,0.75,0,0.02573\n")
    rows = tiles.read_rows(str(ref))
    assert len(rows) == 3 and rows[0]["tc"] == "1" and rows[2]["time_ms"] == "0.02573"
    best = tiles.query_best(rows, 64, 32, 224, 224)
    assert (best["th"], best["tw"], best["tc"]) == ("1", "7", "2")
    assert tiles.load_tables([str(ref)]) == {}                 # no B200 tile fields: nothing to launch from
    own = tiles.load_tables()                                  # the shipped B200 tables
    assert (64, 64, 56, 56, 64, 3, 1) in own and (512, 512, 7, 7, 1, 3, 1) in own
    t = tiles.table_tile(64, 64, 56, 56, 64)
    assert t is not None and t.kc >= 1 and tiles.table_tile(63, 64, 56, 56, 64) is None
    path = os.path.join(ref_import.REFERENCE_ROOT, TABLES["A100"][0])
    if os.path.isfile(path):
        rows = tiles.read_rows(path)
        b = tiles.query_best(rows, 32, 32, 56, 56)
        assert [int(b[k]) for k in ("th", "tw", "tc")] == PICKS["A100"]["shapes"]["32,32,56,56"]["best"]
