"""Generates tests/golden/tkconv_cases.npz and tests/golden/core_cfg1.npz by running the
reference's own, unmodified TKConv2dC (inference/TKConv.py) on CPU.

    python tests/golden/make_golden.py          # needs the reference tree (see oracle/ref_import.py)

Every case draws from torch.Generator().manual_seed(seed): x ~ N(0,1) first, then the
three kernels Kaiming-normal (fan_out, relu — the reference's conv init,
inference/resnet_inet_tt.py:337), then the bias ~ N(0,1).  Stored per case: the inputs,
the parameters and what TKConv2dC.forward_features returned (z1, z2, y), all fp32.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import ref_import  # noqa: E402

# name: (seed, B, C, K, R1, R2, H, W, k, stride, pad, bias)
CASES = {
    "k3_s1_p1_bias":   (11, 2, 16, 24, 8, 12, 9, 11, 3, 1, 1, True),
    "k3_s2_p1":        (12, 3, 8, 8, 4, 4, 7, 7, 3, 2, 1, False),
    "k1_s1_p0_bias":   (13, 2, 12, 20, 5, 7, 6, 5, 1, 1, 0, True),
    "k5_s1_p2_bias":   (14, 1, 6, 10, 3, 9, 13, 13, 5, 1, 2, True),
    "one_pixel":       (15, 1, 3, 4, 2, 3, 1, 1, 1, 1, 0, False),
    "k3_s1_p0_ragged": (16, 2, 5, 7, 33, 3, 10, 6, 3, 1, 0, True),
    "k3_s2_p1_even":   (17, 2, 10, 12, 16, 16, 14, 14, 3, 2, 1, False),
    "k3_7x7_r40":      (18, 5, 20, 20, 40, 40, 7, 7, 3, 1, 1, False),
}


def kaiming_(t, gen):
    fan_out = t.shape[0] * t.shape[2] * t.shape[3]
    return t.normal_(0.0, (2.0 / fan_out) ** 0.5, generator=gen)


def draw(seed, B, C, K, R1, R2, H, W, k, bias):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, C, H, W, generator=g)
    first = kaiming_(torch.empty(R1, C, 1, 1), g)
    core = kaiming_(torch.empty(R2, R1, k, k), g)
    last = kaiming_(torch.empty(K, R2, 1, 1), g)
    b = torch.randn(K, generator=g) if bias else None
    return x, first, core, last, b


def main():
    TK = ref_import.import_tkconv()
    torch.set_num_threads(1)
    out, meta = {}, {}
    for name, (seed, B, C, K, R1, R2, H, W, k, stride, pad, bias) in CASES.items():
        x, first, core, last, b = draw(seed, B, C, K, R1, R2, H, W, k, bias)
        m = TK.TKConv2dC(C, K, k, stride=stride, padding=pad, bias=bias,
                         hp_dict=ref_import.Ranks(layer=[R2, R1]), name="layer")
        with torch.no_grad():
            m.first_kernel.copy_(first); m.core_kernel.copy_(core); m.last_kernel.copy_(last)
            if bias:
                m.bias.copy_(b)
            y, (z1, z2, y2) = m.forward_features(x)
            assert torch.equal(y, m.forward(x)) and torch.equal(y, y2)
        for key, t in dict(x=x, first=first, core=core, last=last, z1=z1, z2=z2, y=y).items():
            out[name + "/" + key] = t.numpy()
        if bias:
            out[name + "/bias"] = b.numpy()
        meta[name] = dict(seed=seed, B=B, C=C, K=K, R1=R1, R2=R2, H=H, W=W, k=k, stride=stride, pad=pad, bias=bias)
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "tkconv_cases.npz"), **out)

    # The reference's CPU-runnable case: one core conv, N=1, R1=R2=32, 56x56, 3x3, s1, p1.
    g = torch.Generator().manual_seed(1001)
    x = torch.randn(1, 32, 56, 56, generator=g)
    core = kaiming_(torch.empty(32, 32, 3, 3), g)
    m = TK.TKConv2dC(32, 32, 3, stride=1, padding=1, bias=False, hp_dict=ref_import.Ranks(layer=[32, 32]), name="layer")
    with torch.no_grad():
        m.core_kernel.copy_(core)
        # identity 1x1 factors: forward_features then exposes the core conv alone
        m.first_kernel.copy_(torch.eye(32).reshape(32, 32, 1, 1))
        m.last_kernel.copy_(torch.eye(32).reshape(32, 32, 1, 1))
        _, (z1, z2, _) = m.forward_features(x)
    assert torch.equal(z1, x)
    np.savez_compressed(os.path.join(HERE, "core_cfg1.npz"), x=x.numpy(), core=core.numpy(), z2=z2.numpy(),
                        torch_version=np.frombuffer(torch.__version__.encode(), dtype=np.uint8))
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
