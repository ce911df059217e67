"""Per-shape layer driver — the run-time counterpart of the reference's generated drivers.

The reference emits one program per shape whose main() fills the input with rand()%10 and the
filter with ones, times cuDNN and one un-warmed launch of its kernel with a cudaEvent pair,
prints `N,C,H,W,<times>,<speedups>,diff` and appends the row to a CSV
(A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:412-514; shapes and
compile loop at compile_run.py:14-52).  Here shape and tile are arguments:

    python -m tdc_b200.layer_driver --shape 64,64,56,56 [--batch 1] [--tile th,tw,tc,tn,nog,gy,gx,imgs,ks]
                                    [--filter 3] [--stride 1] [--pad 1] [--iters 20] [--csv out.csv]

`--shape` is C,N,H,W in the reference's naming (C input, N output channels of the core
conv).  Output row: N,C,H,W,B,cudnn_ms,tdc_first_ms,tdc_ms,speedup,frac_fp32,diff — `diff` is
the reference's L1 check (exact integers expected: 0), `tdc_first_ms` its protocol (first
launch, no warm-up), `tdc_ms` the warmed median.

`--reference-row` prints (and appends to `--csv`) the reference's own row instead,
`N,C,H,W,FFT,WINO,GEMM,TVM,TDC,FFT/TDC,WINO/TDC,GEMM/TDC,TVM/TDC,diff` (template_benchmark_cudnn.template:500-512;
times in ms): the three cuDNN algorithm classes are timed by `cudnn_layer_baseline` (baselines/cudnn_layer.cpp, a
process of its own), TDC is the warmed median of this build's kernel, TVM is `nan` (the AutoTVM baseline is not
reproduced).  `tdc_b200.end2end` reads these rows.
"""
import argparse
import statistics
import sys


def cudnn_algorithm_times(B, C, H, W, K, R, S, pad, stride, iters=20):
    """(fft_ms, winograd_ms, gemm_ms) of cuDNN's three legacy algorithm classes for one layer, from the
    `cudnn_layer_baseline` tool run as a child process; NaN where cuDNN refuses an algorithm or the tool is not
    built."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cudnn_layer_baseline")
    nan = float("nan")
    if not os.path.exists(exe):
        print("cudnn_layer_baseline is not built (python ppopp23-tdc_b200/build.py): cuDNN columns are nan", file=sys.stderr)
        return nan, nan, nan
    r = subprocess.run([exe] + [str(v) for v in (B, C, H, W, K, R, S, pad, stride, iters)], capture_output=True, text=True,
                       timeout=600)
    if r.returncode != 0:
        print("cudnn_layer_baseline failed: %s" % r.stderr.strip(), file=sys.stderr)
        return nan, nan, nan
    fft, wino, gemm = (float(v) for v in r.stdout.strip().split(",")[:3])
    return fft, wino, gemm


def main(argv=None):
    import torch
    import torch.nn.functional as F
    from . import ops
    from ._lib import Tile, W_CRSK

    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", required=True, help="C,N,H,W (reference naming)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--tile", default=None)
    ap.add_argument("--filter", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-cudnn", action="store_true")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--reference-row", action="store_true",
                    help="print the reference's CSV row with the cuDNN FFT / Winograd / implicit-GEMM times")
    ap.add_argument("--tc", type=int, default=0, choices=[0, 1, 3, 4],
                    help="run the tensor-core variant instead: 4 = 3xFP16, 3 = 3xTF32 (both fp32-level), 1 = plain TF32")
    a = ap.parse_args(argv)
    Cc, N, H, W = (int(v) for v in a.shape.split(","))
    B, k = a.batch, a.filter
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream()
    g = torch.Generator().manual_seed(1)
    x = torch.randint(0, 10, (B, Cc, H, W), generator=g).float().to(dev)
    w = torch.ones(Cc, k, k, N, device=dev)
    tile = Tile(*(int(v) for v in a.tile.split(","))) if a.tile else ops.select_tile(B, Cc, H, W, N, k, k, a.pad, a.stride)
    Ho, Wo = ops.out_hw(H, W, k, k, a.pad, a.stride)
    y = torch.empty(B, N, Ho, Wo, device=dev)

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream); fn(); e1.record(stream); e1.synchronize()
        return e0.elapsed_time(e1)

    if a.tc:
        from .tc import TcConv
        conv = TcConv(w, mode=a.tc, w_layout=W_CRSK)
        run = lambda: conv(x, out=y)
    else:
        run = lambda: ops.core_conv2d(x, w, a.stride, a.pad, w_layout=W_CRSK, tile=tile, out=y)
    first = timed(run)
    for _ in range(3):
        run()
    tdc = statistics.median(timed(run) for _ in range(a.iters))
    exact = F.conv2d(x.double(), torch.ones(N, Cc, k, k, device=dev, dtype=torch.double), None, a.stride, a.pad)
    diff = float((y.double() - exact).abs().sum())
    cud = float("nan")
    if not a.no_cudnn:
        torch.backends.cudnn.benchmark = True
        torch.backends.cudnn.allow_tf32 = False
        wk = torch.ones(N, Cc, k, k, device=dev)
        for _ in range(3):
            F.conv2d(x, wk, None, a.stride, a.pad)
        cud = statistics.median(timed(lambda: F.conv2d(x, wk, None, a.stride, a.pad)) for _ in range(a.iters))
    sm = ops.query_device().sm_count
    flops = 2.0 * B * N * Cc * k * k * Ho * Wo
    frac = flops / (tdc * 1e-3) / (sm * 128 * 2 * 1.965e9)
    row = "%d,%d,%d,%d,%d,%f,%f,%f,%f,%f,%g" % (N, Cc, H, W, B, cud, first, tdc, cud / tdc, frac, diff)
    if a.reference_row:
        fft, wino, gemm = cudnn_algorithm_times(B, Cc, H, W, N, k, k, a.pad, a.stride, a.iters)
        tvm = float("nan")
        row = "%d,%d,%d,%d,%f,%f,%f,%f,%f,%f,%f,%f,%f,%g" % (N, Cc, H, W, fft, wino, gemm, tvm, tdc, fft / tdc, wino / tdc,
                                                             gemm / tdc, tvm / tdc, diff)
    print(row)
    print("tile", tile, file=sys.stderr)
    if a.csv:
        with open(a.csv, "a") as f:
            f.write(row + "\n")
    return 0 if diff == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
