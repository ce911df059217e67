#!/usr/bin/env python
"""Benchmark of the Tucker core-convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the core conv over the eight sweep shapes
(H=W, R1=R2) in {(56,32),(56,64),(28,64),(28,128),(14,128),(14,256),(7,256),(7,512)},
3x3, stride 1, pad 1, fp32, batch 64 per GPU (weak scaling: every rank runs its own batch,
no collective on the data path).  Rank 0 prints ONE JSON line.

  value          layer-images/s = (8 layers x 64 images x N GPUs) / time per step, inputs resident in HBM
  e2e            the same work through the layer objects of the C ABI with HOST buffers
                 (tdc_conv_forward_host: copy in, run, copy out), pinned host memory
  roofline       the step's kernel (tcgen05, 3xTF32) against a third of the dense TF32 peak, with its
                 HBM figure; the fp32 FMA kernels against the fp32 FMA peak under `fp32_fma_path`
  cpu_baseline   the reference's CPU path for the same step (torch F.conv2d on the host cores)
  layers         per-shape kernel time at batch 64 and batch 1, and cuDNN through torch
                 (allow_tf32=False) beside it

`--impl reference` times the reference's CPU implementation of the path (the three
F.conv2d calls of inference/TKConv.py:90-95 reduce to the core call for this step) on the
host cores of the box, on the same step: all eight shapes at batch 64.  It is one host whatever
--gpus says (rank 0 runs it, the other ranks exit).
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "ppopp23-tdc_b200"))

SWEEP = [(56, 32, 32), (56, 64, 64), (28, 64, 64), (28, 128, 128), (14, 128, 128), (14, 256, 256),
         (7, 256, 256), (7, 512, 512)]
BATCH = 64
METRIC, UNIT = "core_conv_sweep_throughput", "layer-images/s"
WORKLOAD = "core-conv sweep: 8 shapes (H,R1=R2) 56/32 56/64 28/64 28/128 14/128 14/256 7/256 7/512, 3x3 s1 p1, batch 64 per GPU"


def conv_flops(B, H, R1, R2):
    return 2.0 * B * R2 * R1 * 9 * H * H


def conv_bytes(B, H, R1, R2):
    return 4.0 * (B * R1 * H * H + B * R2 * H * H + R2 * R1 * 9)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], sm_max_mhz=d.get("sm_max_mhz", 1965.0), bf16_tflops=d.get("bf16_tflops", 1590.0),
                    source="measured")
    return dict(hbm_gbs=6650.0, sm_max_mhz=1965.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock/throttle samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.f, self.p = index, None, None

    def __enter__(self):
        try:
            self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None
        return self

    def __exit__(self, *a):
        if self.p is not None:
            self.p.terminate()
            try:
                self.p.wait(timeout=5)
            except Exception:
                self.p.kill()

    def summary(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.f is None:
            return out
        try:
            self.f.flush()
            rows = [r.split(",") for r in open(self.f.name).read().strip().splitlines() if r.count(",") >= 8]
            os.unlink(self.f.name)
        except Exception:
            return out
        if not rows:
            return out
        sm = [float(r[1]) for r in rows]
        out["sm_mhz"] = statistics.median(sm)
        out["sm_max_mhz"] = float(rows[0][2])
        out["power_w_max"] = max(float(r[3]) for r in rows)
        out["samples"] = len(rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for i, n in enumerate(names):
            if any("Active" in r[5 + i] and "Not" not in r[5 + i] for r in rows):
                out["reasons"].append(n)
        return out


def recorded_dram_bytes():
    """{(H, R1): bytes} from the data file that sits beside the ncu summary of the step's launches: lines `H R1 bytes`."""
    out = {}
    path = os.path.join(ROOT, "profiles", "sweep_b64_dram_bytes.txt")
    if os.path.exists(path):
        for ln in open(path):
            f = ln.split()
            if len(f) >= 3 and not ln.startswith("#"):
                out[(int(f[0]), int(f[1]))] = float(f[2])
    return out


def cpu_core_step(torch, batch, threads):
    """The reference's CPU path for one step at `batch` images per layer; returns seconds."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as O
    torch.set_num_threads(threads)
    layers = []
    g = torch.Generator().manual_seed(9)
    for (H, R1, R2) in SWEEP:
        x = torch.randn(batch, R1, H, H, generator=g)
        w = torch.randn(R2, R1, 3, 3, generator=g) * (2.0 / (R2 * 9)) ** 0.5
        layers.append((O.TKConv2dCRef(None, w, None, None, 1, 1), x))

    def step():
        with torch.no_grad():
            for m, x in layers:
                m.core(x)
    return step


def run_reference(args):
    """Reference arm: the CPU implementation of the path on the host cores, bounded sample."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample_b = BATCH                       # the whole step: a pass costs some tens of milliseconds on the host cores
    step = cpu_core_step(torch, sample_b, cores)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = len(SWEEP) * sample_b / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "impl": "torch.nn.functional.conv2d on CPU, the call TKConv2dC.forward makes (inference/TKConv.py:92-93); "
                           "one host with all its cores, whatever --gpus says"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "the whole step: batch %d per layer, all 8 shapes, %d steps" % (sample_b, args.steps)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def torch_reference_forward(torch, m, x):
    """The reference's GPU path for the same network and weights: the three F.conv2d calls of
    TKConv2dC.forward (inference/TKConv.py:90-95) per Tucker conv and the module sequence of
    TTBasicBlock / TTResNet (inference/resnet_inet_tt.py:102-117,380-394), i.e. cuDNN through
    torch.  A reported baseline; none of the product's kernels run here."""
    F = torch.nn.functional

    def conv(c, t):
        if hasattr(c, "first_kernel"):
            t = F.conv2d(t, c.first_kernel)
            t = F.conv2d(t, c.core_kernel, None, c.stride, c.padding)
            return F.conv2d(t, c.last_kernel, c.bias)
        return F.conv2d(t, c.weight, c.bias, c.stride, c.padding)

    def bn(b, t):
        return F.batch_norm(t, b.running_mean, b.running_var, b.weight, b.bias, False, 0.0, b.eps)

    x = F.max_pool2d(F.relu(bn(m.bn1, conv(m.conv1, x))), 3, 2, 1)
    for layer in (m.layer1, m.layer2, m.layer3, m.layer4):
        for blk in layer:
            out = F.relu(bn(blk.bn1, conv(blk.conv1, x)))
            out = bn(blk.bn2, conv(blk.conv2, out))
            idt = x if blk.downsample is None else bn(blk.downsample[1], conv(blk.downsample[0], x))
            x = F.relu(out + idt)
    return m.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def bench_tk_block(torch, T, dev, time_layer, peaks):
    """The whole Tucker block (1x1 C->R1, 3x3 core, 1x1 R2->K) for the ResNet-50 bottleneck middles
    C=K in {64@56, 128@28, 256@14, 512@7}, R1=R2=C/2, at batch 1 and 32, as the module runs it under "auto"
    (`us`; `strategy` says whether that is the three-launch chain or ONE launch with the factors multiplied into
    one filter, which keeps no intermediate at all), as three launches (`us_three_launches`), and through
    torch/cuDNN both as the three convolutions the reference calls and as one dense conv on the same merged
    filter.  `tflops` counts the block's factored FLOPs.  HBM floor: x in + y out + filters once."""
    import torch.nn.functional as F

    class HP:
        ranks = {}
    rows = []
    torch.backends.cudnn.benchmark = True
    torch.backends.cudnn.allow_tf32 = False
    for i, (Cc, H) in enumerate(((64, 56), (128, 28), (256, 14), (512, 7))):
        R = Cc // 2
        HP.ranks = {"b": [R, R]}
        m = T.TKConv2dC_B200(Cc, Cc, 3, padding=1, bias=False, hp_dict=HP, name="b")
        g = torch.Generator().manual_seed(3000 + i)
        x32 = torch.randn(32, Cc, H, H, generator=g)
        with torch.no_grad():
            for p in (m.first_kernel, m.core_kernel, m.last_kernel):
                p.normal_(0.0, (2.0 / (p.shape[0] * p.shape[2] * p.shape[3])) ** 0.5, generator=g)
        m = m.to(dev)
        m.precision = "auto"
        for B in (1, 32):
            x = x32[:B].contiguous().to(dev)
            with torch.no_grad():
                us = time_layer(lambda: m(x), iters=10)
                ref = lambda t: F.conv2d(F.conv2d(F.conv2d(t, m.first_kernel), m.core_kernel, None, 1, 1), m.last_kernel)
                cud = time_layer(lambda: ref(x), iters=10)
                # the same block as three launches (the factored form as written) and, for cuDNN, as one dense conv too
                m.precision = "fp16x3"
                us_chain = time_layer(lambda: m(x), iters=10)
                m.precision = "auto"
                wd = m._dense_weight()
                cud_dense = time_layer(lambda: F.conv2d(x, wd, None, 1, 1), iters=10)
                y64 = ref(x[:2].double()) if False else F.conv2d(F.conv2d(F.conv2d(x[:2].double(), m.first_kernel.double()),
                                                                           m.core_kernel.double(), None, 1, 1), m.last_kernel.double())
                err = float((m(x)[:2].double() - y64).abs().max() / y64.abs().max())
            flops = 2.0 * B * H * H * (Cc * R + 9 * R * R + R * Cc)
            by = 4.0 * (2 * B * Cc * H * H + 2 * Cc * R + 9 * R * R)
            from tdc_b200.dispatch import tucker_strategy
            row = dict(C=Cc, H=H, R=R, B=B, us=us, strategy=tucker_strategy(m, x, "auto"), us_three_launches=us_chain, cudnn_us=cud,
                       cudnn_dense_us=cud_dense, rel_err_fp64=err, tflops=flops / us / 1e6,
                       hbm_floor_us=by / peaks["hbm_gbs"] / 1e3, gbs=by / us / 1e3)
            if B == 1:
                # batch-1 latency without host launch gaps on either side: the three launches replayed from a CUDA graph
                for key, fn in (("graph_us", lambda: m(x)), ("cudnn_graph_us", lambda: ref(x))):
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side), torch.no_grad():
                        for _ in range(3):
                            fn()
                    torch.cuda.current_stream().wait_stream(side)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph), torch.no_grad():
                        fn()
                    for _ in range(3):
                        graph.replay()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(); [graph.replay() for _ in range(50)]; e1.record()
                    torch.cuda.synchronize()
                    row[key] = e0.elapsed_time(e1) * 1e3 / 50
            rows.append(row)
    return rows


def bench_resnet(torch, T, dev, dist, world, rank, stream):
    """images/s of the TK-compressed ResNet-18 (ranks round8(0.5*channels), random init, eval) at
    batch 256 per GPU and its batch-1 latency, with the cuDNN path on the same weights beside it."""
    from tdc_b200.parallel import gather_slices
    model = T.fill_deterministic(T.tkc_resnet18(precision="auto").eval(), seed=0).to(dev)
    out = {}
    with torch.no_grad():
        for B, iters in ((256, 5), (32, 20), (1, 30)):
            x = torch.randn(B, 3, 224, 224, generator=torch.Generator().manual_seed(4001 + rank)).to(dev)

            def fwd():
                y = model(x)
                return gather_slices(y, B * world) if (dist is not None and B > 1) else y
            for _ in range(3):
                y = fwd()
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(iters):
                y = fwd()
            e1.record(stream)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            if dist is not None:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            key = "b%d" % B
            out[key] = {"ms": ms, "images_per_s": B * (world if B > 1 else 1) / (ms * 1e-3)}
            if world == 1:
                torch.backends.cudnn.benchmark = True
                torch.backends.cudnn.allow_tf32 = False
                for _ in range(3):
                    yr = torch_reference_forward(torch, model, x)
                torch.cuda.synchronize()
                e0.record(stream)
                for _ in range(iters):
                    yr = torch_reference_forward(torch, model, x)
                e1.record(stream)
                torch.cuda.synchronize()
                out[key]["cudnn_ms"] = e0.elapsed_time(e1) / iters
                # both against the same network in fp64 on the first images
                nb = min(B, 4)
                y64 = torch_reference_forward(torch, model.double(), x[:nb].double())
                model.float()
                out[key]["rel_err_fp64"] = float((y[:nb].double() - y64).abs().max() / y64.abs().max())
                out[key]["cudnn_rel_err_fp64"] = float((yr[:nb].double() - y64).abs().max() / y64.abs().max())
        if world == 1:
            # batch-1 latency with the whole forward captured in a CUDA graph (launch-bound otherwise)
            x1 = torch.randn(1, 3, 224, 224, generator=torch.Generator().manual_seed(4001)).to(dev)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(3):
                    model(x1)
            torch.cuda.current_stream().wait_stream(s)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                yg = model(x1)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); [graph.replay() for _ in range(30)]; e1.record()
            torch.cuda.synchronize()
            out["b1"]["graph_ms"] = e0.elapsed_time(e1) / 30
            out["b1"]["graph_matches_eager"] = bool(torch.equal(yg, model(x1)))
            # the cuDNN path under a CUDA graph as well, so both sides are free of launch gaps
            with torch.cuda.stream(s):
                for _ in range(3):
                    torch_reference_forward(torch, model, x1)
            torch.cuda.current_stream().wait_stream(s)
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2):
                torch_reference_forward(torch, model, x1)
            for _ in range(3):
                g2.replay()
            torch.cuda.synchronize()
            e0.record(); [g2.replay() for _ in range(30)]; e1.record()
            torch.cuda.synchronize()
            out["b1"]["cudnn_graph_ms"] = e0.elapsed_time(e1) / 30
    out["config"] = "ResNet-18 [2,2,2,2], all sixteen 3x3 convs Tucker with R=round8(0.5*ch), 224x224 N(0,1) images, fp32, eval"
    return out


def torch_densenet_forward(torch, m, x):
    """The reference's GPU path for the TK-DenseNet: torch.cat of all earlier features per layer, BatchNorm + ReLU,
    the bottleneck conv, BatchNorm + ReLU, the three F.conv2d calls of the Tucker conv
    (inference/densenet_inet_tt.py:56-60,103-108,134-139; TKConv.py:90-95), i.e. cuDNN through torch.  A reported
    baseline; none of the product's kernels run here."""
    F = torch.nn.functional

    def conv(c, t):
        if hasattr(c, "first_kernel"):
            t = F.conv2d(t, c.first_kernel)
            t = F.conv2d(t, c.core_kernel, None, c.stride, c.padding)
            return F.conv2d(t, c.last_kernel, c.bias)
        return F.conv2d(t, c.weight, c.bias, c.stride, c.padding)

    def bn_relu(b, t):
        return F.relu(F.batch_norm(t, b.running_mean, b.running_var, b.weight, b.bias, False, 0.0, b.eps))

    f = m.features
    x = F.max_pool2d(bn_relu(f.norm0, conv(f.conv0, x)), 3, 2, 1)
    for name, mod in f.named_children():
        if name.startswith("denseblock"):
            feats = [x]
            for layer in mod.values():
                z = conv(layer.conv1, bn_relu(layer.norm1, torch.cat(feats, 1)))
                feats.append(conv(layer.conv2, bn_relu(layer.norm2, z)))
            x = torch.cat(feats, 1)
        elif name.startswith("transition"):
            x = F.avg_pool2d(conv(mod.conv, bn_relu(mod.norm, x)), 2, 2)
    x = bn_relu(f.norm5, x)
    return m.classifier(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def bench_densenet(torch, T, dev):
    """TK-DenseNet-121 (the reference's shipped ranks: every 3x3 conv Tucker [32, 32]) at batch 1 and 32, each forward
    captured as a CUDA graph — the network is ~300 launches, launch-bound from the interpreter — with the cuDNN path on
    the same weights, also as a graph, beside it."""
    model = T.fill_deterministic(T.tkc_densenet121(precision="auto").eval(), seed=0, gain=0.7).to(dev)
    torch.backends.cudnn.benchmark = True
    torch.backends.cudnn.allow_tf32 = False
    out = {}

    class Ref:
        def eval(self):
            return self

        def __call__(self, t):
            return torch_densenet_forward(torch, model, t)
    with torch.no_grad():
        for B, iters in ((1, 20), (32, 10)):
            x = torch.randn(B, 3, 224, 224, generator=torch.Generator().manual_seed(121)).to(dev)
            row = {}
            for key, net in (("graph_ms", model), ("cudnn_graph_ms", Ref())):
                g = T.GraphedForward(net, x)
                for _ in range(3):
                    g(x)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    y = g(x)
                e1.record()
                torch.cuda.synchronize()
                row[key] = e0.elapsed_time(e1) / iters
                row["y_" + key] = y[:2].double().clone()
            y64 = torch_densenet_forward(torch, model.double(), x[:2].double())
            model.float()
            row["rel_err_fp64"] = float((row.pop("y_graph_ms") - y64).abs().max() / y64.abs().max())
            row["cudnn_rel_err_fp64"] = float((row.pop("y_cudnn_graph_ms") - y64).abs().max() / y64.abs().max())
            row["images_per_s"] = B / (row["graph_ms"] * 1e-3)
            out["b%d" % B] = row
    out["config"] = ("DenseNet-121 (growth 32, blocks 6/12/24/16), the 3x3 conv of all 58 dense layers Tucker with ranks "
                     "[32, 32], 224x224 N(0,1) images, fp32-level results, eval, CUDA graph on both sides")
    return out


def bench_vgg(torch, T, dev, dist, world, rank, stream):
    """TK-compressed VGG-16 (every 3x3 conv but the first Tucker with R = round8(0.5*channels), random init, eval),
    224x224 N(0,1) images: the batch-2048 job sharded over the GPUs, each rank running its 2048/world images as
    chunks of 128 through the same forward (activations of a 2048-image chunk would not be a sensible working set),
    logits gathered once at the end.  Strong scaling by construction: total work is fixed."""
    from tdc_b200.parallel import gather_slices
    F = torch.nn.functional
    model = T.tkc_vgg16(precision="auto").eval().to(dev)
    TOTAL, CHUNK = 2048, 128
    mine = TOTAL // world
    x = torch.randn(CHUNK, 3, 224, 224, generator=torch.Generator().manual_seed(5001 + rank)).to(dev)

    def job():
        outs = [model(x) for _ in range(mine // CHUNK)]
        y = torch.cat(outs)
        return gather_slices(y, TOTAL) if dist is not None else y

    def torch_forward(t):
        for m in model.features:
            if hasattr(m, "first_kernel"):
                t = F.conv2d(F.conv2d(F.conv2d(t, m.first_kernel), m.core_kernel, None, m.stride, m.padding), m.last_kernel, m.bias)
            elif isinstance(m, torch.nn.Conv2d):
                t = F.conv2d(t, m.weight, m.bias, m.stride, m.padding)
            else:
                t = m(t)
        return model.head.fc(torch.flatten(F.adaptive_avg_pool2d(t, 1), 1))
    out = {}
    with torch.no_grad():
        for _ in range(2):
            y1 = model(x)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        y = job()
        e1.record(stream)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out = {"b2048_ms": ms, "images_per_s": TOTAL / (ms * 1e-3), "chunk": CHUNK, "images_per_gpu": mine}
        if world == 1:
            torch.backends.cudnn.benchmark = True
            torch.backends.cudnn.allow_tf32 = False
            for _ in range(2):
                yr = torch_forward(x)
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(2):
                yr = torch_forward(x)
            e1.record(stream)
            torch.cuda.synchronize()
            out["cudnn_chunk_ms"] = e0.elapsed_time(e1) / 2
            out["chunk_ms"] = ms / (mine // CHUNK)
            y64 = torch_forward_double(torch, model, x[:2])
            out["rel_err_fp64"] = float((y1[:2].double() - y64).abs().max() / y64.abs().max())
            out["cudnn_rel_err_fp64"] = float((yr[:2].double() - y64).abs().max() / y64.abs().max())
    out["config"] = "VGG-16 cfg D, twelve of thirteen 3x3 convs Tucker with R=round8(0.5*ch), 224x224 N(0,1) images, fp32, eval; 2048 images over all GPUs"
    return out


def torch_forward_double(torch, model, x):
    """The same VGG forward in fp64 through torch (the arbiter for the end-to-end error)."""
    F = torch.nn.functional
    t = x.double()
    for m in model.features:
        if hasattr(m, "first_kernel"):
            b = None if m.bias is None else m.bias.double()
            t = F.conv2d(F.conv2d(F.conv2d(t, m.first_kernel.double()), m.core_kernel.double(), None, m.stride, m.padding), m.last_kernel.double(), b)
        elif isinstance(m, torch.nn.Conv2d):
            t = F.conv2d(t, m.weight.double(), None if m.bias is None else m.bias.double(), m.stride, m.padding)
        elif isinstance(m, torch.nn.ReLU):
            t = F.relu(t)
        else:
            t = m(t)
    return F.linear(torch.flatten(F.adaptive_avg_pool2d(t, 1), 1), model.head.fc.weight.double(), model.head.fc.bias.double())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip per-layer table, cuDNN and CPU baselines")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import tdc_b200 as T      # raises if libtdc_b200.so is missing: there is no fallback

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        # keep stdout to the one JSON line: NCCL's version banner goes there at the VERSION level
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    stream = torch.cuda.current_stream()

    # ---- resident inputs: x ~ N(0,1), Kaiming-normal weights, seeded on the CPU ------------
    layers = []
    for i, (H, R1, R2) in enumerate(SWEEP):
        g = torch.Generator().manual_seed(2100 + i + 1000 * rank)
        x = torch.randn(BATCH, R1, H, H, generator=g)
        w = torch.randn(R2, R1, 3, 3, generator=g) * (2.0 / (R2 * 9)) ** 0.5
        xd, wk = x.to(dev), w.to(dev)
        layers.append(dict(H=H, R1=R1, R2=R2, x=xd, w=T.permute_weights(wk), wk=wk, y=torch.empty(BATCH, R2, H, H, device=dev),
                           tile=T.best_tile(BATCH, R1, H, H, R2, 3, 3, 1, 1), tc4=T.TcConv(wk, mode=4), tc3=T.TcConv(wk, mode=3), tc1=T.TcConv(wk, mode=1),
                           x_host=x, w_host=w))

    # The step the headline is quoted on: every layer on the fastest path that keeps fp32-level
    # results (1e-5 bar) — at batch 64 that is the tensor-core kernel with operands split into two
    # fp16 parts (3xFP16) for all eight shapes (one launch each; the kernel takes the scale that
    # brings the input into fp16's range from a sample of the input).  Split TF32
    # parts, the fp32 FMA kernels and plain TF32 are timed beside it below.
    def step_one_stream():
        for L in layers:
            L["tc4"](L["x"], out=L["y"])

    # The eight layers of a step are independent of one another, so the step issues them alternately on two streams
    # that fork from and join the timed stream: a layer whose grid does not fill the GPU (113-128 CTAs on 148 SMs for
    # the 14x14 and 7x7 shapes) or whose last round is short runs beside the start of the next one.  The same step on
    # one stream is reported as `ms_per_step_one_stream`.
    lanes = [torch.cuda.Stream(), torch.cuda.Stream()]

    def step():
        fork = torch.cuda.Event()
        fork.record(stream)
        for k, L in enumerate(layers):
            lane = lanes[k & 1]
            if k < 2:
                lane.wait_event(fork)
            with torch.cuda.stream(lane):
                L["tc4"](L["x"], out=L["y"])
        for lane in lanes:
            join = torch.cuda.Event()
            join.record(lane)
            stream.wait_event(join)

    def step_simt():
        for L in layers:
            T.core_conv2d(L["x"], L["w"], 1, 1, w_layout=T.W_CRSK, tile=L["tile"], out=L["y"])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def time_steps(fn, steps, warm):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clk:
            # warm-up under the sampler for at least half a second, so that nvidia-smi (100 ms period)
            # sees the clocks of this load even when the timed steps take only milliseconds
            t_w = time.perf_counter()
            n_w = 0
            while n_w < warm or (args.steps > 2 and time.perf_counter() - t_w < 0.6):   # short runs (profiling) skip the soak
                fn(); n_w += 1
                if n_w % 16 == 0:
                    torch.cuda.synchronize()
            barrier()
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps, clk.summary()

    ms_step, clocks = time_steps(step, args.steps, max(args.warmup, 3))
    ms_step_one, _ = time_steps(step_one_stream, args.steps, 3)
    value = len(SWEEP) * BATCH * world / (ms_step * 1e-3)
    ms_simt, clocks_simt = time_steps(step_simt, max(3, args.steps // 2), 3)

    # ---- per-kernel timing, live, on the launching stream ------------------------------------
    peaks = measured_peaks()
    sm_count = T.query_device().sm_count
    fp32_peak = sm_count * 128 * 2 * peaks["sm_max_mhz"] * 1e6 / 1e12     # TFLOP/s at the max SM clock
    tf32_peak = peaks["bf16_tflops"] / 2.0                                # dense TF32 = half the measured bf16 rate
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def time_layer(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()                        # evict L2 (256 MB > 126 MB) outside the timed pair
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); fn(); b.record(stream)
            b.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return statistics.median(ts)

    per_layer = []
    for L in layers:
        fl, by = conv_flops(BATCH, L["H"], L["R1"], L["R2"]), conv_bytes(BATCH, L["H"], L["R1"], L["R2"])
        ref = torch.nn.functional.conv2d(L["x"][:2].double(), L["wk"].double(), None, 1, 1)
        row = dict(H=L["H"], R1=L["R1"], R2=L["R2"], B=BATCH)
        for name, fn in (("tc4", lambda L=L: L["tc4"](L["x"], out=L["y"])), ("tc3", lambda L=L: L["tc3"](L["x"], out=L["y"])),
                         ("tc1", lambda L=L: L["tc1"](L["x"], out=L["y"])),
                         ("simt", lambda L=L: T.core_conv2d(L["x"], L["w"], 1, 1, w_layout=T.W_CRSK, tile=L["tile"], out=L["y"]))):
            us = time_layer(fn)
            row[name + "_us"] = us
            row[name + "_tflops"] = fl / us / 1e6
            row[name + "_rel_err_fp64"] = float((L["y"][:2].double() - ref).abs().max() / ref.abs().max())
        row["gbs_tc4"] = by / row["tc4_us"] / 1e3
        row["tile_simt"] = list(L["tile"].as_tuple())
        per_layer.append(row)
    tot_fl = sum(conv_flops(BATCH, r["H"], r["R1"], r["R2"]) for r in per_layer)
    tot_by = sum(conv_bytes(BATCH, r["H"], r["R1"], r["R2"]) for r in per_layer)
    dom = max(per_layer, key=lambda r: r["tc4_us"])
    tot_tc4, tot_tc3, tot_simt, tot_tc1 = (sum(r[k] for r in per_layer) for k in ("tc4_us", "tc3_us", "simt_us", "tc1_us"))
    f16_peak = peaks["bf16_tflops"]                                       # dense fp16 = the measured bf16 rate
    # DRAM bytes (read + write) per launch as one ncu capture of this command recorded them (a data file beside the
    # capture's summary; absent or without the shape: null).  Outputs stay in L2 within a launch.
    recorded = recorded_dram_bytes()
    roofline = {
        "bound": "tensor", "achieved": tot_fl / tot_tc4 / 1e6, "peak": f16_peak / 3.0, "unit": "TFLOP/s",
        "frac": tot_fl / tot_tc4 / 1e6 / (f16_peak / 3.0),
        "traffic": recorded.get((dom["H"], dom["R1"])),
        "traffic_note": {"launch": [dom["H"], dom["R1"], dom["R2"]], "unit": "bytes per launch",
                         "algorithmic_bytes": conv_bytes(BATCH, dom["H"], dom["R1"], dom["R2"]),
                         "source": "recorded: dram__bytes_read.sum + dram__bytes_write.sum of the dominant launch in an earlier ncu "
                                   "capture of this command (not measured by this run)"},
        "kernel": "conv_tc_persist_kernel (tcgen05 kind::f16, operands split into two fp16 parts), the 8 launches of a step, L2 flushed before each",
        "peak_source": "algorithmic FLOPs against bf16_tflops/3: the measured cuBLAS bf16 rate of MEASURED_PEAKS.json (%s) as the dense "
                       "fp16 rate, divided by the three fp16 products each fp32-level product costs" % peaks["source"],
        "dominant_launch": {k: dom[k] for k in ("H", "R1", "R2", "tc4_us", "tc4_tflops")},
        "hbm": {"achieved": tot_by / tot_tc4 / 1e3, "peak": peaks["hbm_gbs"], "unit": "GB/s"},
        "vs_fp32_fma_peak": tot_fl / tot_tc4 / 1e6 / fp32_peak,
        "vs_tf32x3_roof": tot_fl / tot_tc4 / 1e6 / (tf32_peak / 3.0),
        "note": "the roof of the fp16-parts path is twice that of the TF32-parts path it replaced (fp16 MMAs contract 16 channels where "
                "TF32 MMAs contract 8): the same achieved rate reads half as high a fraction; vs_tf32x3_roof gives it against the old roof",
        "tf32x3": {"achieved": tot_fl / tot_tc3 / 1e6, "peak": tf32_peak / 3.0, "frac": tot_fl / tot_tc3 / 1e6 / (tf32_peak / 3.0),
                   "note": "the same step with TF32 parts (mode 3) against a third of the dense TF32 rate"},
    }
    simt = {
        "value": len(SWEEP) * BATCH * world / (ms_simt * 1e-3), "unit": UNIT, "ms_per_step": ms_simt,
        "roofline": {"bound": "fp32", "achieved": tot_fl / tot_simt / 1e6, "peak": fp32_peak, "unit": "TFLOP/s",
                     "frac": tot_fl / tot_simt / 1e6 / fp32_peak,
                     "kernel": "conv_f32_kernel (fp32 FMA, bit-reproducible), the 8 launches of a step",
                     "peak_source": "SMs x 128 lanes x 2 x max SM clock from MEASURED_PEAKS.json (%s)" % peaks["source"]},
    }
    tf32 = {"value": len(SWEEP) * BATCH * world / (tot_tc1 * 1e-6), "unit": UNIT, "tolerance": 5e-3,
            "max_rel_err_fp64": max(r["tc1_rel_err_fp64"] for r in per_layer),
            "note": "plain TF32 (one MMA per product), from per-layer timings; reported separately from the fp32-level paths"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "path": "fp32 in / fp32 out; products on tensor cores with operands split into two fp16 parts (3xFP16, inputs scaled "
                           "into fp16's range by a power of two chosen per call), fp32 accumulation; "
                           "max rel. error vs fp64 over the sweep %.1e (bar 1e-5)" % max(r["tc4_rel_err_fp64"] for r in per_layer),
                   "precision": "fp16x3",
                   "l2": "working set of a step (inputs+outputs 288 MB) exceeds the 126 MB L2; per-layer timings flush L2 explicitly",
                   "streams": "the eight independent layers of a step are issued alternately on two streams forked from and joined to "
                              "the timed stream (ms_per_step_one_stream: the same step on one stream)",
                   "parallelism": "batch shards, no collective" if world > 1 else "single GPU"},
        "clocks": clocks, "gpu_launches": len(SWEEP) * args.steps, "roofline": roofline,
        "us_per_layer_b64": ms_step * 1e3 / len(SWEEP), "ms_per_step_one_stream": ms_step_one,
        "fp32_fma_path": simt, "tf32_path": tf32, "tf32x3_path": {"value": len(SWEEP) * BATCH * world / (tot_tc3 * 1e-6), "unit": UNIT,
                                                                  "max_rel_err_fp64": max(r["tc3_rel_err_fp64"] for r in per_layer)},
        "per_layer_b64": per_layer,
    }

    # ---- end to end through the layer objects with HOST buffers (pinned) -------------------
    lib = T.lib
    hosts = []
    for L in layers:
        h = C.c_void_p()
        wk = L["w_host"].contiguous()
        T._lib.check(lib.tdc_conv_create(C.byref(h), BATCH, L["R1"], L["H"], L["H"], L["R2"], 1, 3, 3, 1,
                                         C.c_void_p(wk.data_ptr()), None))
        T._lib.check(lib.tdc_conv_set_precision(h, 4))
        xin = L["x_host"].pin_memory()
        yout = torch.empty(BATCH, L["R2"], L["H"], L["H"]).pin_memory()
        hosts.append((h, xin, yout))
    h2d = sum(x.numel() * 4 for _, x, _ in hosts)
    d2h = sum(y.numel() * 4 for _, _, y in hosts)

    side = [torch.cuda.Stream() for _ in hosts]      # one stream per (independent) layer

    def e2e_step_sync():
        for h, xin, yout in hosts:
            T._lib.check(lib.tdc_conv_forward_host(h, C.c_void_p(xin.data_ptr()), C.c_void_p(yout.data_ptr())))

    def e2e_step():
        # the eight layers of a step are independent: each goes copy in -> conv -> copy out on its own stream, so
        # one layer's copy out overlaps the next one's copy in; the step ends when every stream has drained
        for (h, xin, yout), st in zip(hosts, side):
            T._lib.check(lib.tdc_conv_forward_host_async(h, C.c_void_p(xin.data_ptr()), C.c_void_p(yout.data_ptr()),
                                                         C.c_void_p(st.cuda_stream)))
        for st in side:
            st.synchronize()

    e2e_steps = max(3, min(args.steps, 10))
    timings = {}
    for name, fn in (("sync", e2e_step_sync), ("async", e2e_step)):
        for _ in range(3):
            fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            fn()
        barrier()
        sec = (time.perf_counter() - t0) / e2e_steps
        if dist is not None:
            t = torch.tensor([sec], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        timings[name] = sec
    e2e_s = timings["async"]
    line["e2e"] = {"value": len(SWEEP) * BATCH * world / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d,
                   "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3,
                   "api": "tdc_conv_forward_host_async per layer, each layer on its own stream and, inside the call, in four batch "
                          "chunks on two streams so that copy in, kernel and copy out overlap (pinned host buffers; "
                          "copies inside the timed region; the step ends when all streams have drained)",
                   "one_layer_at_a_time": {"value": len(SWEEP) * BATCH * world / timings["sync"], "ms_per_step": timings["sync"] * 1e3,
                                           "api": "tdc_conv_forward_host per layer (copy in, conv, copy out, synchronise)"}}
    # what the host link allows: the same buffers copied in and out with no kernel between (copy in on one stream,
    # copy out on another, so both directions run at once), as a ceiling for the end-to-end figure
    dev_in = [torch.empty_like(x, device=dev) for _, x, _ in hosts]
    dev_out = [torch.empty_like(y, device=dev) for _, _, y in hosts]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def copies_only():
        with torch.cuda.stream(s_in):
            for d, (_, x, _) in zip(dev_in, hosts):
                d.copy_(x, non_blocking=True)
        with torch.cuda.stream(s_out):
            for d, (_, _, y) in zip(dev_out, hosts):
                y.copy_(d, non_blocking=True)
        s_in.synchronize(); s_out.synchronize()
    for _ in range(2):
        copies_only()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        copies_only()
    barrier()
    copy_s = (time.perf_counter() - t0) / e2e_steps
    if dist is not None:
        t = torch.tensor([copy_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        copy_s = float(t.item())
    line["e2e"]["copy_ceiling"] = {"ms_per_step": copy_s * 1e3, "value": len(SWEEP) * BATCH * world / copy_s, "unit": UNIT,
                                   "gbs_each_way_per_gpu": h2d / copy_s / 1e9,
                                   "note": "pinned-memory copies of the step's inputs and outputs alone, both directions at once, all ranks at once"}
    line["e2e"]["frac_of_copy_ceiling"] = copy_s / e2e_s
    del dev_in, dev_out
    e2e_step()                      # the copies above wrote scratch data over the host outputs: one more real step
    # one parity probe of the end-to-end output against the resident path
    # (the host path runs the batch in chunks, each with a range scale of its own: the same values to rounding, not to the bit)
    y_res = layers[0]["tc4"](layers[0]["x"])
    e2e_diff = float((hosts[0][2].to(dev) - y_res).abs().max() / y_res.abs().max())
    line["e2e"]["matches_resident_path"] = bool(e2e_diff <= 1e-5)
    line["e2e"]["rel_diff_to_resident_path"] = e2e_diff
    for h, _, _ in hosts:
        lib.tdc_conv_destroy(h)

    # ---- TK-compressed ResNet-18 forward (every rank its own batch; one gather of the logits) --
    if not args.no_extras:
        line["tk_resnet18"] = bench_resnet(torch, T, dev, dist, world, rank, stream)
        line["tk_vgg16"] = bench_vgg(torch, T, dev, dist, world, rank, stream)
        if rank == 0 and world == 1:
            line["tk_block"] = bench_tk_block(torch, T, dev, time_layer, peaks)
            line["tk_densenet121"] = bench_densenet(torch, T, dev)

    # ---- extras on rank 0 of a single-GPU run: batch-1 latency, cuDNN, CPU baseline ---------
    if rank == 0 and world == 1 and not args.no_extras:
        import torch.nn.functional as F
        torch.backends.cudnn.benchmark = True
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_tf32 = False
        table = []
        for L, r64 in zip(layers, per_layer):
            H, R1, R2 = L["H"], L["R1"], L["R2"]
            wk = L["wk"]
            x1 = L["x"][:1].contiguous()
            t1 = T.best_tile(1, R1, H, H, R2, 3, 3, 1, 1)
            y1 = torch.empty(1, R2, H, H, device=dev)
            us1_fp32 = time_layer(lambda: T.core_conv2d(x1, L["w"], 1, 1, w_layout=T.W_CRSK, tile=t1, out=y1), iters=20)
            us1_tc4 = time_layer(lambda: L["tc4"](x1, out=y1), iters=20)
            # batch 1 as the dispatch rule runs it: tensor cores where the layer has the tiles and the arithmetic for it
            from tdc_b200 import tc as _tc
            b1_path = "fp16x3" if _tc.worthwhile(1, R1, H, H, R2, 3) else "fp32"
            us1 = us1_tc4 if b1_path == "fp16x3" else us1_fp32
            cud64 = time_layer(lambda: F.conv2d(L["x"], wk, None, 1, 1))
            cud1 = time_layer(lambda: F.conv2d(x1, wk, None, 1, 1), iters=20)
            ref = F.conv2d(L["x"][:2].double(), wk.double(), None, 1, 1)
            cud_err = float((F.conv2d(L["x"], wk, None, 1, 1)[:2].double() - ref).abs().max() / ref.abs().max())
            table.append(dict(H=H, R1=R1, R2=R2, us_b64=r64["tc4_us"], us_b64_tf32x3=r64["tc3_us"], us_b64_fp32_fma=r64["simt_us"], us_b64_tf32=r64["tc1_us"],
                              cudnn_us_b64=cud64, rel_err_fp64_b64=r64["tc4_rel_err_fp64"], cudnn_rel_err_fp64_b64=cud_err,
                              frac_b64=conv_flops(BATCH, H, R1, R2) / r64["tc4_us"] / 1e6 / (f16_peak / 3.0),
                              us_b1=us1, path_b1=b1_path, us_b1_fp32_fma=us1_fp32, us_b1_fp16x3=us1_tc4,
                              frac_fp32_b1=conv_flops(1, H, R1, R2) / us1_fp32 / 1e6 / fp32_peak, cudnn_us_b1=cud1,
                              tile_b1=list(t1.as_tuple())))
        line["layers"] = table
        # what the timing itself costs: a kernel that does nothing, between the same pair of events after the same flush
        one = torch.zeros(1, device=dev)
        line["timing_floor_us"] = {"value": time_layer(lambda: one.add_(1), iters=20),
                                   "note": "a one-element torch kernel in the per-layer harness (events around one launch, L2 flushed before): "
                                           "the part of every us_b1 figure, ours and cuDNN's, that no kernel can remove"}
        gm = lambda v: float(torch.tensor(v).log().mean().exp())
        line["speedup_vs_cudnn_geomean"] = {"b64": gm([r["cudnn_us_b64"] / r["us_b64"] for r in table]),
                                            "b64_tf32x3": gm([r["cudnn_us_b64"] / r["us_b64_tf32x3"] for r in table]),
                                            "b64_fp32_fma_kernels": gm([r["cudnn_us_b64"] / r["us_b64_fp32_fma"] for r in table]),
                                            "b64_tf32": gm([r["cudnn_us_b64"] / r["us_b64_tf32"] for r in table]),
                                            "b1": gm([r["cudnn_us_b1"] / r["us_b1"] for r in table]),
                                            "cudnn": "torch F.conv2d, cudnn.benchmark=True, allow_tf32=False, version %s" % torch.backends.cudnn.version()}
        cores = os.cpu_count() or 1
        cstep = cpu_core_step(torch, BATCH, cores)
        cstep()
        t0 = time.perf_counter()
        n = 0
        while n < 3 or (time.perf_counter() - t0 < 10.0 and n < 50):
            cstep(); n += 1
        cdt = (time.perf_counter() - t0) / n
        line["cpu_baseline"] = {"value": len(SWEEP) * BATCH / cdt, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": "the whole step (batch %d per layer, all 8 shapes), %d passes of torch F.conv2d on CPU" % (BATCH, n)}
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
