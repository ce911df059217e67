"""Writes tests/golden/selector_picks.json by calling the reference's OWN selector functions
(TDC-LAYERS-MODELING/model.py: get_occupancy_dict, get_result_dict, oracl, build_table,
modeling, loss; TDC-LAYERS-ORACLE/gen_from_occupancy.py: query_best) on the reference's own
tables, for both GPU trees.

    python tests/golden/make_selector_golden.py         # needs the reference tree

Stored per GPU and shape: the model pick (th,tw,tc), the table-best pick, both times, and the
mean loss — and, for the three README claims that can be checked from the tables, nothing else.
The tables themselves are not copied.
"""
import importlib.util
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TDC_REFERENCE_ROOT", "/root/reference")


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def one(tree, table_name, sms, thr, ratio):
    model = load(os.path.join(REF, tree, "TDC-LAYERS-MODELING", "model.py"), "ref_model_" + tree[:4])
    gen = load(os.path.join(REF, tree, "TDC-LAYERS-ORACLE", "gen_from_occupancy.py"), "ref_gen_" + tree[:4])
    table = os.path.join(REF, tree, "TDC-LAYERS-MODELING", table_name)
    lines = open(table).readlines()
    shapes = [(64, 32, 224, 224), (64, 32, 112, 112), (32, 32, 56, 56), (64, 32, 56, 56), (64, 64, 56, 56), (32, 32, 28, 28),
              (64, 32, 28, 28), (96, 64, 28, 28), (160, 96, 28, 28), (192, 96, 28, 28), (32, 32, 14, 14), (64, 32, 14, 14),
              (128, 96, 14, 14), (192, 96, 14, 14), (32, 32, 7, 7), (64, 32, 7, 7), (96, 64, 7, 7), (192, 160, 7, 7)]
    occ = model.get_occupancy_dict(lines)
    res = model.get_result_dict(lines)
    orc = model.oracl(table, shapes)
    tab = model.build_table(shapes, occ, sms, thr)
    out, tot = {}, 0.0
    for s in shapes:
        th, tw, tc = model.modeling(tab, s, 0.0, 0.9, 0.1, ratio)
        ls = model.loss(s, th, tw, tc, orc, res)
        best = gen.query_best(s[0], s[1], s[2], s[3], table).split(",")
        out["%d,%d,%d,%d" % s] = {"model": [th, tw, tc], "model_ms": res[s + (th, tw, tc)],
                                  "best": [int(best[-6]), int(best[-5]), int(best[-4])], "best_ms": float(best[-1]), "loss": ls}
        tot += ls
    return {"shapes": out, "mean_loss": tot / len(shapes), "rows": len(lines)}


def main():
    sys.stdout = open(os.devnull, "w")      # the reference functions print
    picks = {"A100": one("A100-evaluation", "a100-occupancy-unrolled", 108, 2048, 0.05),
             "2080Ti": one("2080Ti-evaluation", "2080Ti-occupancy-unrolled", 68, 1024, 0.15)}
    sys.stdout = sys.__stdout__
    json.dump(picks, open(os.path.join(HERE, "selector_picks.json"), "w"), indent=1, sort_keys=True)
    print({k: (v["mean_loss"], v["rows"]) for k, v in picks.items()})


if __name__ == "__main__":
    main()
