"""Makes tc_vs_fp32_times_b200.json (run on a B200): 420 layers — 3x3 and 1x1, 32..2048 channels, 7..56 pixels, batch
1..64 — timed on the tensor-core kernel (fp16 parts, unbiased sums) and on the fp32 FMA kernel with its best tile, L2
flushed before every launch, median of five.  Rows: [R, C, K, H, batch, tensor-core us, fp32 us].  The thresholds of
tdc_b200.tc.worthwhile are a fit to this file; tests/test_dispatch_cpu.py holds the rule to it.

    python tests/golden/make_tc_vs_fp32_times.py [out.json]
"""
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "ppopp23-tdc_b200"))

SHAPES = ((64, 64, 56), (128, 32, 56), (256, 64, 56), (64, 256, 56), (512, 128, 28), (128, 512, 28), (256, 64, 28), (512, 128, 14), (1024, 128, 7),
          (1024, 512, 7), (512, 128, 7), (128, 32, 7), (128, 32, 14), (128, 32, 28), (32, 32, 56), (64, 32, 56), (32, 64, 56), (128, 128, 28),
          (64, 64, 28), (128, 64, 28), (64, 128, 28), (256, 256, 14), (128, 128, 14), (256, 128, 14), (128, 256, 14), (512, 512, 7), (256, 256, 7),
          (512, 256, 7), (256, 512, 7), (1024, 256, 14), (256, 1024, 14), (2048, 512, 7), (512, 2048, 7))


def main(out_path):
    import torch
    import tdc_b200 as T
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn, iters=5):
        for _ in range(2):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return statistics.median(ts)

    rows = []
    for R in (3, 1):
        for (C, K, H) in SHAPES:
            if R == 3 and max(C, K) > 512:
                continue
            for B in (1, 2, 4, 8, 16, 32, 64):
                g = torch.Generator().manual_seed(1)
                x = torch.randn(B, C, H, H, generator=g).to(dev)
                w = (torch.randn(K, C, R, R, generator=g) * 0.05).to(dev)
                y = torch.empty(B, K, H, H, device=dev)
                conv = T.TcConv(w, mode=4, unbiased=True)
                t_tc = timeit(lambda: conv(x, out=y))
                wc, tile = T.permute_weights(w), T.best_tile(B, C, H, H, K, R, R, (R - 1) // 2, 1)
                t_fp = timeit(lambda: T.core_conv2d(x, wc, 1, (R - 1) // 2, w_layout=T.W_CRSK, tile=tile, out=y))
                rows.append([R, C, K, H, B, round(t_tc, 1), round(t_fp, 1)])
    with open(out_path, "w") as f:
        f.write("[\n" + ",\n".join(json.dumps(r) for r in rows) + "\n]\n")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "tc_vs_fp32_times_b200.json"))
