"""TK-compressed ResNet-18: key compatibility with the reference (CPU) and output parity with
the reference's own TTResNet run on CPU (GPU; golden logits in tests/golden/tk_resnet18.npz)."""
import os

import numpy as np
import pytest
import torch

from helpers import GOLDEN, NET_FP32_TOL, NET_TC_TOL, rel_err

Z = np.load(os.path.join(GOLDEN, "tk_resnet18.npz"))


def test_state_dict_keys_and_ranks_match_the_reference(built):
    import tdc_b200 as T
    m = T.tkc_resnet18()
    assert sorted(m.state_dict().keys()) == list(Z["keys"])
    hp = T.HalfRanks()
    assert hp.ranks["layer1.0.conv1.weight"] == [32, 32] and hp.ranks["layer2.0.conv1.weight"] == [64, 32]
    assert hp.ranks["layer4.1.conv2.weight"] == [256, 256] and len(hp.ranks) == 16
    assert tuple(m.layer2[0].conv1.core_kernel.shape) == (64, 32, 3, 3) and m.layer2[0].conv1.stride == (2, 2)
    assert sum(p.numel() for p in m.parameters()) == 4714024
    with pytest.raises(T.TdcError):
        m.train()(torch.zeros(1, 3, 224, 224))


def test_hp_dict_selects_which_convs_are_tucker(built):
    import tdc_b200 as T

    class HP:
        ranks = {"layer1.0.conv1.weight": [16, 24]}
    m = T.TKResNet((1, 1, 1, 1), hp_dict=HP)
    assert isinstance(m.layer1[0].conv1, T.TKConv2dC_B200) and m.layer1[0].conv1.in_rank == 24
    assert isinstance(m.layer1[0].conv2, torch.nn.Conv2d) and isinstance(m.layer2[0].conv1, torch.nn.Conv2d)


@pytest.mark.gpu
def test_logits_match_the_reference_network(built):
    import tdc_b200 as T
    m = T.fill_deterministic(T.tkc_resnet18().eval(), seed=0).cuda()
    x = torch.randn(2, 3, 224, 224, generator=torch.Generator().manual_seed(4001)).cuda()
    feats = {}
    m.layer1.register_forward_hook(lambda mod, i, o: feats.__setitem__("layer1", o))
    m.layer4.register_forward_hook(lambda mod, i, o: feats.__setitem__("layer4", o))
    with torch.no_grad():
        logits = m(x)
    # sixteen Tucker blocks deep, BatchNorm folded into the convs, on the fp32 FMA kernels: the whole network is held
    # to the bar of a single layer (the golden logits are the reference network's own fp32 run on the CPU)
    assert rel_err(feats["layer1"][0].mean((1, 2)).cpu().numpy(), Z["layer1_mean"]) <= NET_FP32_TOL
    assert rel_err(feats["layer4"][0].mean((1, 2)).cpu().numpy(), Z["layer4_mean"]) <= NET_FP32_TOL
    assert rel_err(logits.cpu().numpy(), Z["logits"]) <= NET_FP32_TOL
    assert (logits.argmax(1).cpu().numpy() == Z["logits"].argmax(1)).all()


@pytest.mark.gpu
def test_fused_epilogue_against_separate_ops(built):
    import tdc_b200 as T
    g = torch.Generator().manual_seed(9)
    x = torch.randn(3, 16, 14, 14, generator=g).cuda()
    w = (torch.randn(24, 16, 3, 3, generator=g) * 0.1).cuda()
    scale, shift = (torch.rand(24, generator=g) + 0.5).cuda(), torch.randn(24, generator=g).cuda()
    res = torch.randn(3, 24, 14, 14, generator=g).cuda()
    y = T.conv2d_epi(x, w, scale, shift, res, True, 1, 1)
    ref = torch.relu(torch.nn.functional.conv2d(x.double(), w.double(), padding=1) * scale.double().view(1, -1, 1, 1)
                     + shift.double().view(1, -1, 1, 1) + res.double())
    assert rel_err(y.cpu().numpy(), ref.cpu().numpy()) <= 1e-5
    with pytest.raises(T.TdcError):
        T.conv2d_epi(x, w, scale, shift, res[:, :, :7], True, 1, 1)


Z50 = np.load(os.path.join(GOLDEN, "tk_resnet50.npz"))


def test_resnet50_keys_and_ranks_match_the_reference(built):
    """Bottleneck assembly (reference: TTBottleneck / tkc_resnet50): state-dict keys equal to those of the reference's
    own TTResNet(TTBottleneck, [3,4,6,3], conv=TKConv2dC) (tests/golden/make_golden_resnet50.py), the 3x3 conv of every
    block Tucker, the stride on that conv."""
    import tdc_b200 as T
    m = T.tkc_resnet50()
    assert sorted(m.state_dict().keys()) == list(Z50["keys"])
    hp = T.HalfRanksBottleneck()
    assert len(hp.ranks) == 16 and hp.ranks["layer3.5.conv2.weight"] == [128, 128]
    b = m.layer2[0]
    assert isinstance(b.conv2, T.TKConv2dC_B200) and b.conv2.stride == (2, 2) and tuple(b.conv2.core_kernel.shape) == (64, 64, 3, 3)
    assert isinstance(b.conv1, torch.nn.Conv2d) and tuple(b.conv1.weight.shape) == (128, 256, 1, 1)
    assert tuple(b.downsample[0].weight.shape) == (512, 256, 1, 1) and m.fc.in_features == 2048
    assert sum(p.numel() for p in m.parameters()) == 18326568


@pytest.mark.gpu
@pytest.mark.parametrize("precision", ["fp32", "auto"])
def test_resnet50_logits_match_the_reference_network(built, precision):
    import tdc_b200 as T
    m = T.fill_deterministic(T.tkc_resnet50(precision=precision).eval(), seed=0).cuda()
    x = torch.randn(2, 3, 128, 128, generator=torch.Generator().manual_seed(4050)).cuda()
    feats = {}
    m.layer1.register_forward_hook(lambda mod, i, o: feats.__setitem__("layer1", o))
    m.layer4.register_forward_hook(lambda mod, i, o: feats.__setitem__("layer4", o))
    with torch.no_grad():
        logits = m(x)
    # 53 chained convolutions: the fp32 kernels at the single-layer bar, the tensor-core tier at its own
    tol = NET_FP32_TOL if precision == "fp32" else NET_TC_TOL
    assert rel_err(feats["layer1"][0].mean((1, 2)).cpu().numpy(), Z50["layer1_mean"]) <= tol
    assert rel_err(feats["layer4"][0].mean((1, 2)).cpu().numpy(), Z50["layer4_mean"]) <= tol
    assert rel_err(logits.cpu().numpy(), Z50["logits"]) <= tol
    assert (logits.argmax(1).cpu().numpy() == Z50["logits"].argmax(1)).all()
