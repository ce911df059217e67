"""Measured tile table for B200 — the counterpart of the reference's occupancy/time tables.

The reference builds `a100-occupancy-unrolled` by generating, compiling and running one
program per (shape, th, tw, tc) (A100-evaluation/Gen-occupancy/gen.py:78-102,
template.cu:231-287) and picks the fastest row per shape
(A100-evaluation/TDC-LAYERS-ORACLE/gen_from_occupancy.py:51-66).  Here the kernel takes its
tile at run time, so the table is built in one process:

    python -m tdc_b200.tune --batch 64 --out table.csv [--shapes sweep|resnet18] [--max-per-shape 300]

Rows keep the reference's ten columns `C,N,H,W,th,tw,tc,occupancy,diff,time_ms` (C/N =
input/output channels of the core conv) and append the fields this kernel adds:
`B,tn,nog,gy,gx,imgs,ks,threads,smem,ctas,model_cycles,kc,R,stride`.  `diff` is the L1 distance to the
exact result for integer inputs 0..9 and all-ones weights, the reference drivers' own check
(template_benchmark_cudnn.template:418-428,509); it must be 0 in every row.
`best_rows(path)` is query_best() for such a table.
"""
import argparse
import csv
import itertools
import random
import statistics
import sys

SWEEP = [(56, 32, 32), (56, 64, 64), (28, 64, 64), (28, 128, 128), (14, 128, 128), (14, 256, 256),
         (7, 256, 256), (7, 512, 512)]
COLUMNS = ["C", "N", "H", "W", "th", "tw", "tc", "occupancy", "diff", "time_ms",
           "B", "tn", "nog", "gy", "gx", "imgs", "ks", "threads", "smem", "ctas", "model_cycles", "kc", "R", "stride"]


def cdiv(a, b):
    return (a + b - 1) // b


def resnet18_shapes():
    """(C, N, H, W, R, stride, pad) of every convolution of the TK-compressed ResNet-18 with
    ranks round8(0.5*channels): stem, Tucker 1x1 / core / 1x1 triples, 1x1 stride-2 downsamples."""
    shapes = [(3, 64, 224, 224, 7, 2, 3)]
    inpl, H = 64, 56
    for planes in (64, 128, 256, 512):
        stride = 1 if planes == 64 else 2
        for blk in range(2):
            cin = inpl if blk == 0 else planes
            s = stride if blk == 0 else 1
            r1, r2 = 8 * round(0.5 * cin / 8), 8 * round(0.5 * planes / 8)
            Ho = H // s
            shapes += [(cin, r1, H, H, 1, 1, 0), (r1, r2, H, H, 3, s, 1), (r2, planes, Ho, Ho, 1, 1, 0)]      # conv1
            shapes += [(planes, r2, Ho, Ho, 1, 1, 0), (r2, r2, Ho, Ho, 3, 1, 1), (r2, planes, Ho, Ho, 1, 1, 0)]  # conv2
            if blk == 0 and (s != 1 or cin != planes):
                shapes.append((cin, planes, H, H, 1, s, 0))
            H = Ho
        inpl = planes
    seen, out = set(), []
    for sh in shapes:
        if sh not in seen:
            seen.add(sh); out.append(sh)
    return out


def resnet50_shapes():
    """(C, N, H, W, R, stride, pad) of every convolution of the TK-compressed ResNet-50 (bottleneck blocks [3,4,6,3], the
    3x3 conv of every block Tucker with R1 = R2 = round8(0.5*width), the stride on that conv): stem, per block the 1x1
    reduce, the Tucker conv's three steps, the 1x1 expand, and the 1x1 downsample convs."""
    shapes = [(3, 64, 224, 224, 7, 2, 3)]
    inpl, H = 64, 56
    for planes, n, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
        r = 8 * round(0.5 * planes / 8)
        for blk in range(n):
            s = stride if blk == 0 else 1
            Ho = H // s
            shapes += [(inpl, planes, H, H, 1, 1, 0), (planes, r, H, H, 1, 1, 0), (r, r, H, H, 3, s, 1), (r, planes, Ho, Ho, 1, 1, 0),
                       (planes, 4 * planes, Ho, Ho, 1, 1, 0)]
            if blk == 0:
                shapes.append((inpl, 4 * planes, H, H, 1, s, 0))
            inpl, H = 4 * planes, Ho
    seen, out = set(), []
    for sh in shapes:
        if sh not in seen:
            seen.add(sh); out.append(sh)
    return out


def sweep_shapes():
    return [(R1, R2, H, H, 3, 1, 1) for (H, R1, R2) in SWEEP]


def tkblock_shapes():
    """The three convolutions of the Tucker blocks C = K in {64@56, 128@28, 256@14, 512@7}, R1 = R2 = C/2
    (the middles of the ResNet-50 bottlenecks): 1x1 C->R, 3x3 R->R, 1x1 R->C."""
    out = []
    for C, H in ((64, 56), (128, 28), (256, 14), (512, 7)):
        R = C // 2
        out += [(C, R, H, H, 1, 1, 0), (R, R, H, H, 3, 1, 1), (R, C, H, H, 1, 1, 0)]
    return out


def densenet121_shapes(block_config=(6, 12, 24, 16), growth=32, bn_size=4):
    """Every convolution of TK-DenseNet-121 with the reference's shipped ranks (inference/hp_dicts/tk_densenet121_hp.py):
    the stem, per dense layer the 1x1 bottleneck conv (C0 + i*growth -> 128) and the Tucker conv's three steps
    (128 -> 32 1x1, 32 -> 32 3x3, 32 -> 32 1x1), and the three transition convs."""
    shapes = [(3, 2 * growth, 224, 224, 7, 2, 3)]
    c, H = 2 * growth, 56
    mid = bn_size * growth
    for s, n in enumerate(block_config):
        for i in range(n):
            shapes.append((c + i * growth, mid, H, H, 1, 1, 0))
        shapes += [(mid, growth, H, H, 1, 1, 0), (growth, growth, H, H, 3, 1, 1), (growth, growth, H, H, 1, 1, 0)]
        c += n * growth
        if s != len(block_config) - 1:
            shapes.append((c, c // 2, H, H, 1, 1, 0))
            c, H = c // 2, H // 2
    return shapes


def candidates(B, C, H, W, K, R=3, S=3, pad=1, stride=1):
    """Every tile of the compiled thread-tile set that can be launched for the shape."""
    Ho, Wo = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    out = []
    exact = (R, stride) in ((3, 1), (3, 2), (1, 1))
    families = ((4, 4, (8, 16)), (8, 2, (4, 8)), (4, 2, (8, 16)), (8, 1, (4, 8)), (4, 1, (4, 8))) if exact else \
               ((8, 1, (4, 8)), (4, 1, (4, 8)))      # other filters run on the run-time-size instances (one row per thread)
    tiles = [(tn, th, tw, nog) for (tn, th, nogs) in families for tw in (7, 8) for nog in nogs]
    for tn, th, tw, nog in tiles:
        if tn * nog > max(K, 16) * 2:
            continue
        maxt = 256 if tn * th * tw > 64 else 512
        GY, GX = cdiv(Ho, th), cdiv(Wo, tw)
        gys = sorted({cdiv(GY, n) for n in range(1, GY + 1)})
        gxs = sorted({cdiv(GX, n) for n in range(1, GX + 1)})
        for gy, gx in itertools.product(gys, gxs):
            ims = [1]
            if gy == GY and gx == GX:
                ims += [m for m in (2, 3, 4, 6, 7, 8, 12, 14, 16) if m <= B]
            for im in ims:
                nt = nog * im * gy * gx
                for ks in (1, 2, 4, 8):
                    thr = nt * ks
                    if thr > maxt or thr < (64 if B > 1 else 32):
                        continue
                    for tc in (4, 8, 16, 32):
                        if tc % ks or tc > max(C, 8) or (tc == 4 and C > 16):
                            continue
                        tiles_n = cdiv(K, tn * nog) * cdiv(Ho, gy * th) * cdiv(Wo, gx * tw) * cdiv(B, im)
                        for kc in ((1, 2, 4, 8) if tiles_n < 296 else (1,)):
                            if kc == 1 or cdiv(C, tc) >= kc:
                                out.append((th, tw, tc, tn, nog, gy, gx, im, ks, kc))
    return out


def best_rows(path):
    """Fastest row per (C,N,H,W,B,R,stride): the reference's query_best over this table."""
    best = {}
    with open(path) as f:
        for row in csv.DictReader(f):
            if float(row["diff"]) != 0.0:
                continue
            key = tuple(int(row[k]) for k in ("C", "N", "H", "W", "B")) + (int(row.get("R") or 3), int(row.get("stride") or 1))
            if key not in best or float(row["time_ms"]) < float(best[key]["time_ms"]):
                best[key] = row
    return best


def main(argv=None):
    import torch
    from . import ops
    from ._lib import Tile, TdcError, W_CRSK

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--out", default="tile_table.csv")
    ap.add_argument("--shapes", default="sweep", choices=["sweep", "resnet18", "resnet50", "tkblock", "densenet121"])
    ap.add_argument("--shape-list", default=None,
                    help="shapes of one's own instead of a named set: C,N,H,W,R,stride,pad;C,N,H,W,R,stride,pad;...")
    ap.add_argument("--max-per-shape", type=int, default=300)
    ap.add_argument("--model-top", type=int, default=60,
                    help="candidates the analytical model ranks best are always measured, beside the random sample")
    ap.add_argument("--keep", default=None, help="an earlier table: its tile for a shape is measured again beside the new candidates")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--best-out", default=None, help="also write the fastest row per shape to this CSV")
    a = ap.parse_args(argv)
    rnd = random.Random(a.seed)
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream()
    cover = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    reps = 1 if a.batch >= 16 else 8
    if a.shape_list:
        shapes = [tuple(int(v) for v in item.split(",")) for item in a.shape_list.split(";") if item.strip()]
        if any(len(sh) != 7 for sh in shapes):
            ap.error("--shape-list items are C,N,H,W,R,stride,pad")
    else:
        shapes = {"sweep": sweep_shapes, "resnet18": resnet18_shapes, "resnet50": resnet50_shapes, "tkblock": tkblock_shapes, "densenet121": densenet121_shapes}[a.shapes]()
    kept = best_rows(a.keep) if a.keep else {}
    with open(a.out, "w", newline="") as f:
        wr = csv.writer(f)
        wr.writerow(COLUMNS)
        for (Cc, N, H, W, R, stride, pad) in shapes:
            B = a.batch
            shape = (B, Cc, H, W, N, R, R, pad, stride)
            g = torch.Generator().manual_seed(H * 1000 + Cc)
            x = torch.randint(0, 10, (B, Cc, H, W), generator=g).float().to(dev)
            w = torch.ones(Cc, R, R, N, device=dev)
            exact = torch.nn.functional.conv2d(x.double(), torch.ones(N, Cc, R, R, device=dev, dtype=torch.double),
                                               None, stride, pad).float()
            y = torch.empty_like(exact)
            cands = candidates(B, Cc, H, W, N, R, R, pad, stride)
            model_pick = ops.select_tile(*shape).as_tuple()
            if len(cands) > a.max_per_shape:
                def modelled(c):
                    try:
                        return ops.tile_cost(shape, Tile(*c))[0]
                    except TdcError:
                        return float("inf")
                ranked = sorted(cands, key=modelled)[:a.model_top]
                cands = ranked + [c for c in rnd.sample(cands, a.max_per_shape) if c not in ranked]
            if model_pick not in cands:
                cands.append(model_pick)
            old = kept.get((Cc, N, H, W, B, R, stride))
            if old is not None:
                old = tuple(int(old[k]) for k in ("th", "tw", "tc", "tn", "nog", "gy", "gx", "imgs", "ks", "kc"))
                if old not in cands:
                    cands.append(old)
            n_ok = 0
            for c in cands:
                t = Tile(*c)
                try:
                    info = ops.tile_info(shape, t)
                    cost, _ = ops.tile_cost(shape, t)
                    run = lambda: ops.core_conv2d(x, w, stride, pad, w_layout=W_CRSK, tile=t, out=y)
                    run(); run()
                    ts = []
                    for _ in range(a.iters):
                        # a memset keeps the GPU busy while the host enqueues, so the event pair
                        # brackets `reps` back-to-back launches and no host launch latency
                        cover.zero_()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        for _ in range(reps):
                            run()
                        e1.record(stream); e1.synchronize()
                        ts.append(e0.elapsed_time(e1) / reps)
                    diff = float((y - exact).abs().sum())
                except TdcError:
                    continue
                n_ok += 1
                occ = info.ctas_per_sm * info.threads / 2048.0
                wr.writerow([Cc, N, H, W, t.th, t.tw, t.tc, "%.4f" % occ, "%g" % diff, "%.6f" % statistics.median(ts),
                             B, t.tn, t.nog, t.gy, t.gx, t.imgs, t.ks, info.threads, info.smem_bytes, info.grid_x,
                             "%.0f" % cost, t.kc, R, stride])
            f.flush()
            print("shape", (Cc, N, H, W, R, stride), "rows", n_ok, "model pick", model_pick, file=sys.stderr)
    best = best_rows(a.out)
    for key, row in sorted(best.items()):
        print(key, "best %.4f ms" % float(row["time_ms"]),
              {k: row[k] for k in ("th", "tw", "tc", "tn", "nog", "gy", "gx", "imgs", "ks", "kc")}, file=sys.stderr)
    if a.best_out:
        with open(a.best_out, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=COLUMNS)
            wr.writeheader()
            for key, row in sorted(best.items()):
                wr.writerow(row)


if __name__ == "__main__":
    main()
