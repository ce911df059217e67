"""TK-compressed VGG-16 feature stack: reference key layout (CPU) and parity with the same
assembly run through torch on the CPU (GPU)."""
import pytest
import torch

from helpers import NET_FP32_TOL, NET_TC_TOL, NET_TF32X3_TOL, rel_err


def torch_forward(m, x):
    """The reference's path for this assembly: nn.Sequential order of TenVGG.features
    (inference/vgg_tt.py:113-136) with TKConv2dC.forward's three F.conv2d calls (TKConv.py:90-95)."""
    F = torch.nn.functional
    for mod in m.features:
        if hasattr(mod, "first_kernel"):
            x = F.conv2d(F.conv2d(F.conv2d(x, mod.first_kernel), mod.core_kernel, None, mod.stride, mod.padding),
                         mod.last_kernel, mod.bias)
        elif isinstance(mod, torch.nn.Conv2d):
            x = F.conv2d(x, mod.weight, mod.bias, mod.stride, mod.padding)
        else:
            x = mod(x)
    return m.head.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def test_keys_follow_the_reference_numbering(built):
    import tdc_b200 as T
    hp = T.HalfRanksVGG()
    assert sorted(hp.ranks, key=lambda k: int(k.split(".")[1])) == ["features.%d.weight" % i for i in
                                                                    (2, 5, 7, 10, 12, 14, 17, 19, 21, 24, 26, 28)]
    assert hp.ranks["features.2.weight"] == [32, 32] and hp.ranks["features.5.weight"] == [64, 32]
    m = T.tkc_vgg16()
    keys = list(m.state_dict())
    assert keys[:2] == ["features.0.weight", "features.0.bias"]
    assert keys[2:6] == ["features.2.first_kernel", "features.2.core_kernel", "features.2.last_kernel", "features.2.bias"]
    assert keys[-2:] == ["head.fc.weight", "head.fc.bias"]
    # the batch-norm variant lands on the keys of inference/hp_dicts/tk_vgg16_bn_hp.py
    hpb = T.HalfRanksVGG(batch_norm=True)
    assert sorted(int(k.split(".")[1]) for k in hpb.ranks) == [3, 7, 10, 14, 17, 20, 24, 27, 30, 34, 37, 40]
    mb = T.tkc_vgg16(batch_norm=True)
    assert isinstance(mb.features[3], T.TKConv2dC_B200) and isinstance(mb.features[0], torch.nn.Conv2d)
    with pytest.raises(T.TdcError):
        m.eval()(torch.zeros(1, 3, 32, 32))


@pytest.mark.gpu
@pytest.mark.parametrize("bn", [False, True])
def test_vgg16_matches_torch_assembly(built, bn):
    import tdc_b200 as T
    m = T.fill_deterministic(T.tkc_vgg16(batch_norm=bn).eval(), seed=3)
    x = torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(5001))
    with torch.no_grad():
        ref = torch_forward(m, x)
        m = m.cuda()
        y = m(x.cuda())
        m.precision = "tf32x3"
        y3 = m(x.cuda())
        m.precision = "fp16x3"
        y4 = m(x.cuda())
    assert rel_err(y.cpu().numpy(), ref.numpy()) <= NET_FP32_TOL        # 13 convs (37 launches) deep, fp32 FMA kernels
    assert rel_err(y3.cpu().numpy(), ref.numpy()) <= NET_TF32X3_TOL and rel_err(y4.cpu().numpy(), ref.numpy()) <= NET_TC_TOL
