"""Generates tests/golden/tk_resnet18.npz by running the reference's own TTResNet
(inference/resnet_inet_tt.py, unmodified, with TKConv2dC as its conv class) on CPU.

    python tests/golden/make_golden_resnet.py        # needs the reference tree

Network: TTResNet(TTBasicBlock, [2,2,2,2], conv=TKConv2dC) with ranks
[round8(.5*out), round8(.5*in)] for all sixteen 3x3 convs, eval mode, every parameter and
buffer set by tdc_b200.resnet.fill_deterministic (seeded by tensor name, so the B200 model
with the same state-dict keys gets the same values).  Input: 2 images 3x224x224 ~ N(0,1) from
torch.Generator().manual_seed(4001).  Stored: the logits, and the outputs of layer1 and layer4
for image 0 (channel means, to localise a mismatch).
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
    from tdc_b200.resnet import HalfRanks, fill_deterministic
    torch.set_num_threads(8)
    model = R.TTResNet(R.TTBasicBlock, [2, 2, 2, 2], conv=TK.TKConv2dC, hp_dict=HalfRanks()).eval()
    fill_deterministic(model, seed=0)
    x = torch.randn(2, 3, 224, 224, generator=torch.Generator().manual_seed(4001))
    feats = {}
    model.layer1.register_forward_hook(lambda m, i, o: feats.__setitem__("layer1", o))
    model.layer4.register_forward_hook(lambda m, i, o: feats.__setitem__("layer4", o))
    with torch.no_grad():
        logits = model(x)
    np.savez_compressed(os.path.join(HERE, "tk_resnet18.npz"), logits=logits.numpy(),
                        layer1_mean=feats["layer1"][0].mean((1, 2)).numpy(),
                        layer4_mean=feats["layer4"][0].mean((1, 2)).numpy(),
                        keys=np.array(sorted(model.state_dict().keys())))
    print("logits", logits.shape, float(logits.abs().max()), "params", sum(p.numel() for p in model.parameters()))


if __name__ == "__main__":
    main()
