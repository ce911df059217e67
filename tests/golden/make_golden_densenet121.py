"""Generates tests/golden/tk_densenet121.npz by running the reference's own TenDenseNet
(inference/densenet_inet_tt.py:36-281, unmodified, TKConv2dC as its conv class) on CPU with the reference's shipped
rank dictionary (inference/hp_dicts/tk_densenet121_hp.py: the 3x3 conv of every dense layer Tucker, ranks [32, 32]).

    python tests/golden/make_golden_densenet121.py        # needs the reference tree

timm is not installed here; oracle/ref_import.import_densenet says which two timm building blocks are restated
(BatchNorm2d + ReLU, and the average-pool classifier head) — the dense layers, blocks, transitions and Tucker convs
are the reference's code.  Network: growth 32, blocks (6, 12, 24, 16), eval mode, every parameter and buffer set by
tdc_b200.resnet.fill_deterministic (conv gain 0.7: with 58 concatenating layers the plain Kaiming fill
overflows the logits, a smaller one lets the stem drown the dense layers).  Input: 2 images 3x112x112 ~ N(0,1) from torch.Generator().manual_seed(121)
(smaller than the benchmark's 224 to keep the CPU run and the GPU test short; the last block then runs on 3x3 maps,
the odd-sized path of the elementwise and pooling kernels).  Stored: the logits, channel means of the first dense
block's and of the final feature map of image 0, the state-dict keys, and the rank dictionary's keys.

A second, smaller network has SVD 1x1 convs as well (ranks 16 on the first two bottleneck convs of block 1 and on
transition 1) to cover the SVDConv2dC branches of TenDenseLayer / TenDenseTransition (:41-47,149-155).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.join(HERE, "..", "..")
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "ppopp23-tdc_b200"))
import ref_import  # noqa: E402

SVD_RANKS = {"features.denseblock1.denselayer1.conv1.weight": [16], "features.denseblock1.denselayer2.conv1.weight": 16,
             "features.transition1.conv.weight": [16]}


def small_ranks():
    """Rank dictionary of the second network: blocks (2, 2), every 3x3 conv Tucker [32, 32], three SVD 1x1 convs."""
    from tdc_b200.densenet import Growth32Ranks
    hp = Growth32Ranks((2, 2), 32)
    hp.ranks.update(SVD_RANKS)
    return hp


def main():
    D = ref_import.import_densenet()
    TK = ref_import.import_tkconv()
    hp = ref_import.import_hp_dict("tk_densenet121_hp").HyperParamsDictRatio2x
    from tdc_b200.resnet import fill_deterministic
    torch.set_num_threads(8)
    model = D.TenDenseNet(32, (6, 12, 24, 16), conv=TK.TKConv2dC, hp_dict=hp).eval()
    fill_deterministic(model, seed=0, gain=0.7)
    x = torch.randn(2, 3, 112, 112, generator=torch.Generator().manual_seed(121))
    feats = {}
    model.features.denseblock1.register_forward_hook(lambda m, i, o: feats.__setitem__("block1", o))
    model.features.norm5.register_forward_hook(lambda m, i, o: feats.__setitem__("final", o))
    with torch.no_grad():
        logits = model(x)
        small = D.TenDenseNet(32, (2, 2), conv=TK.TKConv2dC, hp_dict=small_ranks()).eval()
        fill_deterministic(small, seed=1)
        xs = torch.randn(3, 3, 64, 64, generator=torch.Generator().manual_seed(122))
        small_logits = small(xs)
    np.savez_compressed(os.path.join(HERE, "tk_densenet121.npz"), logits=logits.numpy(),
                        block1_mean=feats["block1"][0].mean((1, 2)).numpy(),
                        final_mean=feats["final"][0].mean((1, 2)).numpy(),
                        keys=np.array(sorted(model.state_dict().keys())), rank_keys=np.array(sorted(hp.ranks.keys())),
                        small_logits=small_logits.numpy(), small_keys=np.array(sorted(small.state_dict().keys())))
    print("logits", logits.shape, float(logits.abs().max()), "small", float(small_logits.abs().max()),
          "params", sum(p.numel() for p in model.parameters()))


if __name__ == "__main__":
    main()
