"""End-to-end aggregation in the reference's terms, with measured numbers beside the derived ones.

The reference never runs its own kernel inside a network.  Its end-to-end figure is DERIVED
(A100-evaluation/EndToEnd/build_run.py:48-53,96-113): the measured time of the cuDNN skeleton, minus, for every
core-conv shape of the network, count x (cuDNN-GEMM time - TDC time) taken from the per-layer CSVs
(`<machine>-layers-eval-{oracle,modeling}.csv`, rows `N,C,H,W,FFT,WINO,GEMM,TVM,TDC,...`, times in ms,
template_benchmark_cudnn.template:500-512), and it prints one header line and one value line per network
(build_run.py:168-230).  This module reads those CSVs unchanged (and the ones `tdc_b200.layer_driver` writes in
the same format), applies the same formula, and — because here the kernels do run inside the networks — puts
the MEASURED forward time next to it.

    python -m tdc_b200.end2end --layers layers.csv --network resnet18 --batch 1 [--skeleton-ms 1.17]
"""
import argparse
import csv
import sys


def read_layer_csv(path):
    """{(C, N, H, W): {"fft","wino","gemm","tvm","tdc"}} in ms.  Positional, as the reference reads it
    (build_run.py:62-76): N first, C second (its N = output channels, C = input channels)."""
    out = {}
    with open(path, newline="") as f:
        for parts in csv.reader(f):
            if len(parts) < 9:
                continue
            try:
                n, c, h, w = (int(float(v)) for v in parts[:4])
            except ValueError:
                continue                      # header line
            def num(v):
                try:
                    return float(v)
                except ValueError:
                    return float("nan")
            out[(c, n, h, w)] = dict(fft=num(parts[4]), wino=num(parts[5]), gemm=num(parts[6]), tvm=num(parts[7]), tdc=num(parts[8]))
    return out


def derived_time(skeleton_ms, counts, layers, ours="tdc", base="gemm"):
    """skeleton time - sum over shapes of count x (base - ours): compute_saving() and its use, build_run.py:48-53,
    105-113.  Shapes missing from the CSV raise KeyError, as there."""
    return skeleton_ms - sum(n * (layers[s][base] - layers[s][ours]) for s, n in counts.items())


def core_conv_counts(model, x):
    """{(C, N, H, W): count} of the core convolutions a TK network runs on input `x` (C/N = input/output rank):
    what the reference keeps as hand-written dicts per network (build_run.py:41-46), read off the model instead by
    propagating the image size through TKResNet / TKVGG (no kernel runs)."""
    import torch.nn as nn
    from .tkconv import TKConv2dC_B200
    counts = {}
    H, W = x.shape[2], x.shape[3]

    def out_hw(h, w, k, s, p):
        return (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1

    def visit(m, h, w):
        if isinstance(m, TKConv2dC_B200):
            key = (m.in_rank, m.out_rank, h, w)
            counts[key] = counts.get(key, 0) + 1
        return out_hw(h, w, m.kernel_size[0], m.stride[0], m.padding[0])
    if hasattr(model, "layer1"):                       # TKResNet
        H, W = visit(model.conv1, H, W)
        mp = model.maxpool
        H, W = out_hw(H, W, mp.kernel_size, mp.stride, mp.padding)
        for layer in (model.layer1, model.layer2, model.layer3, model.layer4):
            for blk in layer:
                h1, w1 = visit(blk.conv1, H, W)
                H, W = visit(blk.conv2, h1, w1)
    else:                                              # TKVGG
        for m in model.features:
            if isinstance(m, nn.MaxPool2d):
                H, W = out_hw(H, W, m.kernel_size, m.stride, m.padding)
            elif hasattr(m, "kernel_size") and not isinstance(m, (nn.ReLU, nn.BatchNorm2d)):
                H, W = visit(m, H, W)
    return counts


def report(name, values):
    """The reference's two print lines for one network (build_run.py:168-178): `values` is an ordered
    {column: ms}."""
    header = ",".join("%s(Run time)" % k for k in values)
    line = ",".join("%s(ms)" % v for v in values.values())
    return header + "\n" + line


def main(argv=None):
    import torch
    import tdc_b200 as T
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", required=True, help="per-layer CSV in the reference's row format")
    ap.add_argument("--network", default="resnet18", choices=["resnet18", "vgg16"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--skeleton-ms", type=float, default=None, help="measured time of the cuDNN skeleton; measured here through torch if absent")
    a = ap.parse_args(argv)
    dev = torch.device("cuda")
    model = (T.tkc_resnet18 if a.network == "resnet18" else T.tkc_vgg16)(precision="auto").eval().to(dev)
    x = torch.randn(a.batch, 3, 224, 224, device=dev)
    layers = read_layer_csv(a.layers)
    counts = core_conv_counts(model, x)
    missing = [k for k in counts if k not in layers]
    if missing:
        print("no CSV row for core shapes %s: they are left out of the derived figure" % missing, file=sys.stderr)
    have = {k: v for k, v in counts.items() if k in layers}

    def timed(fn, iters=20):
        with torch.no_grad():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    measured = timed(lambda: model(x))
    name = a.network + "-tk"
    values = {}
    if a.skeleton_ms is not None:
        values[name] = a.skeleton_ms
        values[name + "-derived"] = derived_time(a.skeleton_ms, have, layers)
    values[name + "-measured"] = measured
    print(report(name, values))


if __name__ == "__main__":
    main()
