"""Times one kernel of the library alone and prints its bandwidth (and, for a convolution, its arithmetic rate).

    python kernel_bench.py affine  --batch 32 --channels 224 --of 256 --size 56
    python kernel_bench.py maxpool --batch 256 --channels 64 --size 112      # 3x3 / stride 2 / pad 1
    python kernel_bench.py maxpool2 --batch 128 --channels 64 --size 224     # 2x2 / stride 2
    python kernel_bench.py conv --mode 4 --batch 64 --channels 64 --size 56 [--filter 3]   # core conv, channels -> channels
                                                        # --mode 0: fp32 FMA kernel (table tile), 1 / 3 / 4: tensor cores
    python kernel_bench.py conv --mode 4 --batch 32 --channels 3 --out-channels 64 --size 224 --filter 7 --stride 2 --pad 3
                                                        # a strided layer (here the ResNet stem) on the gathering plans

    python kernel_bench.py phases [--batch 64] [--level 1]  # where a launch of the tensor-core kernel spends its time, per sweep layer

`phases` builds the measurement variant of the library (build.py: build_profile, -DTDC_TC_PROFILE=level), loads it in
place of the normal one and, for each of the eight sweep layers (mode 4, no epilogue options), prints the averages over
the CTAs that had a tile: the time from the start of a CTA to the end of its set-up, to its first full stage, to the end
of its first MMA issuer and to its last barrier (clocks / the SM clock read through nvidia-smi while it runs), and the
issuer's shares: waiting for accumulators, waiting for a full stage, issuing (which blocks while the tensor core's
queue is full) and the rest.  Level 1 leaves the kernel's timing as it is; level 2 adds every role's waits.

`affine`: scale, shift and ReLU over the first `--channels` channels of a [batch][--of][size][size] buffer, the
pre-activation of a DenseNet layer.  Algorithmic bytes = input read once + output written once; the L2 is flushed
before every timed launch (a 256 MB memset), times are CUDA events on the launching stream, median of `--iters`.
"""
import argparse
import os
import statistics
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "ppopp23-tdc_b200"))


def phases(argv):
    """See the module docstring."""
    import ctypes
    import subprocess
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["phases"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--level", type=int, default=1, choices=[1, 2])
    a = ap.parse_args(argv)
    import importlib.util
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("tdc_build", os.path.join(here, "ppopp23-tdc_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    os.environ["TDC_B200_LIB"] = mod.build_profile(a.level)
    import torch
    import tdc_b200 as T
    lib = T.lib
    lib.tdc_tc_profile_read.argtypes = [ctypes.POINTER(ctypes.c_ulonglong), ctypes.c_int]
    dev = torch.device("cuda")
    buf = (ctypes.c_ulonglong * 24)()
    names = ["ld:free stage", "ld:raw slot", "pr:free raw slot", "is:accumulators", "is:full stage", "ep:accumulators", "ld:index work",
             "ep:stores", "ld:convert", "ld:hand-over"]
    role_of = [0, 0, 1, 2, 2, 3, 0, 3, 0, 0]
    for H, C in ((56, 32), (56, 64), (28, 64), (28, 128), (14, 128), (14, 256), (7, 256), (7, 512)):
        g = torch.Generator().manual_seed(1)
        x = torch.randn(a.batch, C, H, H, generator=g).to(dev)
        w = (torch.randn(C, C, 3, 3, generator=g) * (2.0 / (C * 9)) ** 0.5).to(dev)
        conv, y = T.TcConv(w, mode=4), torch.empty(a.batch, C, H, H, device=dev)
        for _ in range(3):
            conv(x, out=y)
        torch.cuda.synchronize()
        lib.tdc_tc_profile_read(buf, 1)
        reps = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            conv(x, out=y)
        e1.record()
        mhz = float(subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits", "-i", str(torch.cuda.current_device())],
                                   capture_output=True, text=True).stdout.split()[0])
        torch.cuda.synchronize()
        lib.tdc_tc_profile_read(buf, 1)
        for _ in range(reps):                    # one launch at a time: a CTA that starts under the launch before it would count its wait for it
            conv(x, out=y)
            torch.cuda.synchronize()
        lib.tdc_tc_profile_read(buf, 1)
        v = list(buf)
        ctas = max(1, v[20])
        us = lambda clocks: clocks / ctas / mhz
        tot = max(1, v[14])
        print("3x3 %3d -> %3d at %2dx%2d, batch %d: %.1f us per launch back to back (SM clock %d MHz); per CTA (%d with a tile): set-up done %.1f us, "
              "first full stage %.1f (producer's first copy issued %.1f, loaders' first index work done %.1f, first raw block landed %.1f), first issuer done %.1f, last barrier %.1f | issuer: waits for accumulators %.1f %%, for a full stage %.1f %%, "
              "issues %.1f %% (%.0f clocks per stage use), rest %.1f %%" % (
                  C, C, H, H, a.batch, e0.elapsed_time(e1) * 1e3 / reps, mhz, ctas // reps, us(v[16]), us(v[17]), us(v[21]), us(v[22]), us(v[23]), us(v[18]), us(v[19]),
                  100.0 * v[3] / tot, 100.0 * v[4] / tot, 100.0 * v[10] / tot, v[10] / max(1, v[11]), 100.0 * (tot - v[3] - v[4] - v[10]) / tot), flush=True)
        if a.level >= 2:
            print("    shares within a role: " + ", ".join("%s %.0f %%" % (names[i], 100.0 * v[i] / v[12 + role_of[i]]) for i in range(10) if v[12 + role_of[i]] and v[i]), flush=True)
    return 0


def main(argv=None):
    if (argv if argv is not None else sys.argv[1:])[:1] == ["phases"]:
        return phases(argv if argv is not None else sys.argv[1:])
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
