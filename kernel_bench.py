"""Times one kernel of the library alone and prints its bandwidth (and, for a convolution, its arithmetic rate).

    python kernel_bench.py affine  --batch 32 --channels 224 --of 256 --size 56
    python kernel_bench.py maxpool --batch 256 --channels 64 --size 112      # 3x3 / stride 2 / pad 1
    python kernel_bench.py maxpool2 --batch 128 --channels 64 --size 224     # 2x2 / stride 2
    python kernel_bench.py conv --mode 4 --batch 64 --channels 64 --size 56 [--filter 3]   # core conv, channels -> channels
                                                        # --mode 0: fp32 FMA kernel (table tile), 1 / 3 / 4: tensor cores
    python kernel_bench.py conv --mode 4 --batch 32 --channels 3 --out-channels 64 --size 224 --filter 7 --stride 2 --pad 3
                                                        # a strided layer (here the ResNet stem) on the gathering plans

`affine`: scale, shift and ReLU over the first `--channels` channels of a [batch][--of][size][size] buffer, the
pre-activation of a DenseNet layer.  Algorithmic bytes = input read once + output written once; the L2 is flushed
before every timed launch (a 256 MB memset), times are CUDA events on the launching stream, median of `--iters`.
"""
import argparse
import os
import statistics
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "ppopp23-tdc_b200"))


def main(argv=None):
    import torch
    import tdc_b200 as T
    from tdc_b200 import ops
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["affine", "maxpool", "maxpool2", "conv"])
    ap.add_argument("--mode", type=int, default=4, choices=[0, 1, 3, 4])
    ap.add_argument("--filter", type=int, default=3)
    ap.add_argument("--out-channels", type=int, default=None, help="output channels of the conv (default: --channels)")
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=None, help="padding of the conv (default: (filter - 1) / 2)")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--channels", type=int, default=224)
    ap.add_argument("--of", type=int, default=None, help="channels of the buffer the input is a prefix of (affine)")
    ap.add_argument("--size", type=int, default=56)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peak-gbs", type=float, default=None, help="measured copy bandwidth to quote the fraction of")
    a = ap.parse_args(argv)
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    B, C, H = a.batch, a.channels, a.size
    if a.kernel == "affine":
        buf = torch.randn(B, a.of or C, H, H, device=dev)
        scale, shift = torch.rand(C, device=dev) + 0.5, torch.randn(C, device=dev)
        out = torch.empty(B, C, H, H, device=dev)
        run = lambda: ops.affine_relu(buf[:, :C], scale, shift, relu=True, out=out)
        nbytes = 2 * out.numel() * 4
    elif a.kernel == "conv":
        k, K, st = a.filter, a.out_channels or C, a.stride
        pad = (k - 1) // 2 if a.pad is None else a.pad
        Ho = (H + 2 * pad - k) // st + 1
        g = torch.Generator().manual_seed(1)
        x = torch.randn(B, C, H, H, generator=g).to(dev)
        w = (torch.randn(K, C, k, k, generator=g) * (2.0 / (C * k * k)) ** 0.5).to(dev)
        out = torch.empty(B, K, Ho, Ho, device=dev)
        general = not (k in (1, 3) and pad == (k - 1) // 2 and (st == 1 or k == 1))
        if a.mode:
            conv = T.TcConv(w, mode=a.mode, general=general)
            kw = dict(stride=st, padding=pad) if general else dict(stride=st)
            run = lambda: conv(x, out=out, **kw)
        else:
            wc, tile = T.permute_weights(w), T.best_tile(B, C, H, H, K, k, k, pad, st)
            run = lambda: T.core_conv2d(x, wc, st, pad, w_layout=T.W_CRSK, tile=tile, out=out)
        nbytes = (x.numel() + out.numel() + w.numel()) * 4
        flops = 2.0 * B * C * K * k * k * Ho * Ho
    else:
        x = torch.randn(B, C, H, H, device=dev)
        k, s, p = (3, 2, 1) if a.kernel == "maxpool" else (2, 2, 0)
        out = ops.pool2d(x, k, s, p)
        run = lambda: ops.pool2d(x, k, s, p, out=out)
        nbytes = (x.numel() + out.numel()) * 4
    for _ in range(3):
        run()
    ts = []
    for _ in range(a.iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream); run(); e1.record(stream); e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    t = statistics.median(ts)
    gbs = nbytes / t / 1e9
    frac = "" if a.peak_gbs is None else "  %.2f of %.1f GB/s" % (gbs / a.peak_gbs, a.peak_gbs)
    extra = "  %.1f TFLOP/s (mode %d)" % (flops / t / 1e12, a.mode) if a.kernel == "conv" else ""
    print("%s: %.1f us, %.1f MB, %.1f GB/s%s%s" % (a.kernel, t * 1e6, nbytes / 1e6, gbs, frac, extra))


if __name__ == "__main__":
    main()
