"""Generates tests/golden/tk_resnet50.npz by running the reference's own TTResNet with bottleneck blocks
(inference/resnet_inet_tt.py:155-237,287-394, unmodified, TKConv2dC as its conv class) on CPU.

    python tests/golden/make_golden_resnet50.py        # needs the reference tree

Network: TTResNet(TTBottleneck, [3,4,6,3], conv=TKConv2dC) with the 3x3 conv of every block Tucker
(ranks [round8(.5*width)] * 2, tdc_b200.resnet.HalfRanksBottleneck), 1x1 convs dense, eval mode, every parameter
and buffer set by tdc_b200.resnet.fill_deterministic.  Input: 2 images 3x128x128 ~ N(0,1) from
torch.Generator().manual_seed(4050) (a smaller image than the benchmark's keeps this CPU run and the GPU test short;
the network is fully convolutional up to its global pool).  Stored: the logits, channel means of layer1 and layer4 of
image 0, and the state-dict keys.
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


def main():
    R = ref_import.import_resnet()
    TK = ref_import.import_tkconv()
    from tdc_b200.resnet import HalfRanksBottleneck, fill_deterministic
    torch.set_num_threads(8)
    model = R.TTResNet(R.TTBottleneck, [3, 4, 6, 3], conv=TK.TKConv2dC, hp_dict=HalfRanksBottleneck()).eval()
    fill_deterministic(model, seed=0)
    x = torch.randn(2, 3, 128, 128, generator=torch.Generator().manual_seed(4050))
    feats = {}
    model.layer1.register_forward_hook(lambda m, i, o: feats.__setitem__("layer1", o))
    model.layer4.register_forward_hook(lambda m, i, o: feats.__setitem__("layer4", o))
    with torch.no_grad():
        logits = model(x)
    np.savez_compressed(os.path.join(HERE, "tk_resnet50.npz"), logits=logits.numpy(),
                        layer1_mean=feats["layer1"][0].mean((1, 2)).numpy(),
                        layer4_mean=feats["layer4"][0].mean((1, 2)).numpy(),
                        keys=np.array(sorted(model.state_dict().keys())))
    print("logits", logits.shape, float(logits.abs().max()), "params", sum(p.numel() for p in model.parameters()))


if __name__ == "__main__":
    main()
