"""Shared pieces of the parity tests: seeded inputs, the error metric, golden loading."""
import json
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# The fp32 bar: max|y - y_ref| / max|y_ref| <= 1e-5 per tensor (the hot path's stated
# tolerance). Both sides are fp32 sums of up to 4608 products in different orders, so
# element-wise relative error is not meaningful near zero crossings; the tensor's own
# largest magnitude is the scale.
FP32_TOL = 1e-5

# Whole networks (16 to 120 convolutions in a chain), max|logits - ref| / max|ref|: the same bar as a single layer on
# every precision.  The fp32 FMA kernels ("fp32") land near 3e-7.  On the tensor-core paths ("auto", "fp16x3", "tf32x3")
# the tensor core rounds its running sum towards zero at every accumulation, a shrink of the same sign in every layer
# that would add up over a chain (1.8e-5 on TK-ResNet-18, 2.5e-5 on TK-VGG-16 with fp16 parts); the networks therefore
# run their convolutions with the expected loss put back (TDC_TC_UNBIASED), which leaves 2e-6 .. 5e-6.
NET_FP32_TOL = 1e-5
NET_TC_TOL = 1e-5
NET_TF32X3_TOL = 1e-5


def rel_err(y, ref):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    scale = np.abs(ref).max()
    return float(np.abs(y - ref).max() / (scale if scale > 0 else 1.0))


def kaiming_(t, gen):
    fan_out = t.shape[0] * t.shape[2] * t.shape[3]
    return t.normal_(0.0, (2.0 / fan_out) ** 0.5, generator=gen)


def draw_core(seed, B, R1, R2, H, W, k=3):
    """x ~ N(0,1) first, then the core kernel Kaiming-normal (fan_out), from one seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, R1, H, W, generator=g)
    w = kaiming_(torch.empty(R2, R1, k, k), g)
    return x, w


def draw_block(seed, B, C, K, R1, R2, H, W, k=3, bias=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, C, H, W, generator=g)
    first = kaiming_(torch.empty(R1, C, 1, 1), g)
    core = kaiming_(torch.empty(R2, R1, k, k), g)
    last = kaiming_(torch.empty(K, R2, 1, 1), g)
    b = torch.randn(K, generator=g) if bias else None
    return x, first, core, last, b


def load_cases():
    z = np.load(os.path.join(GOLDEN, "tkconv_cases.npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    cases = {}
    for name, m in meta.items():
        d = {k: z[name + "/" + k] for k in ("x", "first", "core", "last", "z1", "z2", "y")}
        d["bias"] = z[name + "/bias"] if m["bias"] else None
        d["meta"] = m
        cases[name] = d
    return cases


def load_cfg1():
    z = np.load(os.path.join(GOLDEN, "core_cfg1.npz"))
    return z["x"], z["core"], z["z2"]


# (H=W, R1, R2) of the benchmark sweep; 3x3, stride 1, pad 1; batch 1 and 64.
SWEEP = [(56, 32, 32), (56, 64, 64), (28, 64, 64), (28, 128, 128), (14, 128, 128), (14, 256, 256),
         (7, 256, 256), (7, 512, 512)]
