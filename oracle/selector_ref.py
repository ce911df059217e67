"""CPU restatement of the reference's two tile selectors — TEST INFRASTRUCTURE ONLY.

* `query_best`  — A100-evaluation/TDC-LAYERS-ORACLE/gen_from_occupancy.py:51-66,159-169: the
  rows of a measured table whose text contains "C,N,H,W", fastest one wins; its
  (th, tw, tc) are columns -6, -5, -4.
* `modeling`    — A100-evaluation/TDC-LAYERS-MODELING/model.py:103-234: occupancy and time
  dictionaries keyed by (C,N,H,W,th,tw,tc), the volume / latency table, and the choice: walk
  th, tw in 1..12 and tc in {1,2,4,8,16,32} in that order, keep the FIRST ceil(ratio*len)
  candidates, and take the one with the least a*K + b*I + c*O.  The slice comes before the
  sort, so the flops*waves term never takes part — kept as the reference has it.

Table rows are `C,N,H,W,th,tw,tc,occupancy,diff,time_ms` without a header line
(A100-evaluation/Gen-occupancy/template.cu:278-285).  Pinned by tests/golden/selector_picks.json,
which tests/golden/make_selector_golden.py writes by calling the reference's own functions on
the reference's own tables.
"""
import math

SHAPES = [(64, 32, 224, 224), (64, 32, 112, 112), (32, 32, 56, 56), (64, 32, 56, 56), (64, 64, 56, 56), (32, 32, 28, 28),
          (64, 32, 28, 28), (96, 64, 28, 28), (160, 96, 28, 28), (192, 96, 28, 28), (32, 32, 14, 14), (64, 32, 14, 14),
          (128, 96, 14, 14), (192, 96, 14, 14), (32, 32, 7, 7), (64, 32, 7, 7), (96, 64, 7, 7), (192, 160, 7, 7)]
# (num_sm, threads per SM, a, b, c, ratio): model.py:264-277 of the A100 tree, :265-278 of the 2080Ti tree
A100 = (108, 2048, 0.0, 0.9, 0.1, 0.05)
TI2080 = (68, 1024, 0.0, 0.9, 0.1, 0.15)


def read_lines(path):
    with open(path) as f:
        return [ln for ln in f.read().splitlines() if ln.strip()]


def query_best(lines, c, n, h, w):
    needle = "%d,%d,%d,%d" % (c, n, h, w)
    best, best_t = None, 10000.0
    for ln in lines:
        if needle in ln:                      # substring match, as the reference does
            t = float(ln.split(",")[-1])
            if t < best_t:
                best, best_t = ln, t
    parts = best.split(",")
    return int(parts[-6]), int(parts[-5]), int(parts[-4]), best_t


def _dicts(lines):
    occ, res = {}, {}
    for ln in lines:
        p = ln.split(",")
        key = tuple(int(v) for v in p[:7])
        occ[key] = float(p[-3])
        res[key] = float(p[-1])
    return occ, res


def _latency(C, N, H, W, th, tw, tc, sms, thr_sm, occ):
    flops = (th + 2) * (tw + 2) * tc * 9
    bnum = math.ceil(H / th) * math.ceil(C / tc)
    bdim = math.ceil(W / tw) * N
    one_wave = math.floor(sms * thr_sm * occ[(C, N, H, W, th, tw, tc)] / bdim)
    return flops * math.ceil(bnum / one_wave)


def build_table(shapes, occ, sms, thr_sm):
    table = {}
    for (C, N, H, W) in shapes:
        for th in range(1, 13):
            for tw in range(1, 13):
                for tc in (1, 2, 4, 8, 16):
                    key = (C, N, H, W, th, tw, tc)
                    if th >= H or tw >= W or key not in occ:
                        continue
                    bnum = math.ceil(H / th) * math.ceil(W / tw) * math.ceil(C / tc)
                    K = 9 * tc * N * bnum
                    I = math.ceil(H / th) * (th + 2) * (W + 2) * C
                    O = th * tw * N * bnum
                    table[key] = (K, I, O, _latency(C, N, H, W, th, tw, tc, sms, thr_sm, occ))
    return table


def modeling(table, shape, a, b, c, ratio):
    C, N, H, W = shape
    cands = []
    for th in range(1, 13):
        for tw in range(1, 13):
            for tc in (1, 2, 4, 8, 16, 32):
                key = (C, N, H, W, th, tw, tc)
                if th >= H or tw >= W or key not in table:
                    continue
                K, I, O, flops = table[key]
                cands.append((th, tw, tc, K * a + I * b + O * c, flops))
    head = cands[0:math.ceil(len(cands) * ratio)]
    head.sort(key=lambda v: v[-2])
    return head[0][:3]


def replay(lines, consts, shapes=SHAPES):
    """{shape: {"model": (th,tw,tc), "model_ms", "best": (th,tw,tc), "best_ms", "loss"}} and the mean loss."""
    sms, thr, a, b, c, ratio = consts
    occ, res = _dicts(lines)
    table = build_table(shapes, occ, sms, thr)
    out, tot = {}, 0.0
    for s in shapes:
        th, tw, tc = modeling(table, s, a, b, c, ratio)
        bth, btw, btc, bt = query_best(lines, *s)
        # the reference's "oracl": fastest time among the rows matched by the same substring test
        ms = res[s + (th, tw, tc)]
        out[s] = {"model": (th, tw, tc), "model_ms": ms, "best": (bth, btw, btc), "best_ms": bt, "loss": ms / bt - 1}
        tot += ms / bt - 1
    return out, tot / len(shapes)
