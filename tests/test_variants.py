"""TKConv2dM / TKConv2dR equivalents and the load-time Tucker factorisation."""
import numpy as np
import pytest
import torch

import oracle as O
import ref_import
from helpers import FP32_TOL, rel_err


class HP:
    ranks = {"l": [12, 8]}


def test_partial_tucker_properties(built):
    from tdc_b200.tucker import partial_tucker_hosvd, tucker_to_dense
    g = torch.Generator().manual_seed(0)
    # a filter of exact multilinear rank (6, 5) is recovered exactly
    core0, a, b = torch.randn(6, 5, 3, 3, generator=g), torch.randn(20, 6, generator=g), torch.randn(16, 5, generator=g)
    w = torch.einsum("abrs,ka,cb->kcrs", core0, a, b)
    core, (last, first) = partial_tucker_hosvd(w, [6, 5])
    assert core.shape == (6, 5, 3, 3) and last.shape == (20, 6) and first.shape == (16, 5)
    assert torch.allclose(last.t() @ last, torch.eye(6), atol=1e-5) and torch.allclose(first.t() @ first, torch.eye(5), atol=1e-5)
    assert rel_err(tucker_to_dense(core, last, first).numpy(), w.numpy()) < 1e-5
    # a full-rank filter: the iteration does not do worse than its truncated-SVD start
    w = torch.randn(24, 16, 3, 3, generator=g)
    core, (last, first) = partial_tucker_hosvd(w, [12, 8])
    err = torch.linalg.norm(tucker_to_dense(core, last, first) - w) / torch.linalg.norm(w)
    u0 = torch.linalg.svd(w.reshape(24, -1).double(), full_matrices=False)[0][:, :12]
    u1 = torch.linalg.svd(w.permute(1, 0, 2, 3).reshape(16, -1).double(), full_matrices=False)[0][:, :8]
    start = torch.einsum("kcrs,ka,cb->abrs", w.double(), u0, u1)
    err0 = torch.linalg.norm(torch.einsum("abrs,ka,cb->kcrs", start, u0, u1) - w.double()) / torch.linalg.norm(w.double())
    assert 0 < float(err) <= float(err0) + 1e-6 < 1


def test_module_surfaces(built):
    import tdc_b200 as T
    from tdc_b200.tkconv_variants import TKConv2dM_B200, TKConv2dR_B200
    m = TKConv2dM_B200(16, 24, 3, padding=1, hp_dict=HP, name="l")
    assert [(k, tuple(v.shape)) for k, v in m.state_dict().items()] == \
        [("first_factor", (8, 16)), ("core_kernel", (12, 8, 3, 3)), ("last_factor", (24, 12)), ("bias", (24,))]
    r = TKConv2dR_B200(16, 24, 3, padding=1, hp_dict=HP, name="l")
    assert [(k, tuple(v.shape)) for k, v in r.state_dict().items()] == \
        [("first_factor", (8, 16)), ("core_tensor", (12, 8, 3, 3)), ("last_factor", (24, 12)), ("bias", (24,))]
    if ref_import.available():            # same keys and shapes as the reference's own classes
        TK = ref_import.import_tkconv()
        ref = TK.TKConv2dM(16, 24, 3, padding=1, hp_dict=HP, name="l")
        assert [(k, tuple(v.shape)) for k, v in ref.state_dict().items()] == [(k, tuple(v.shape)) for k, v in m.state_dict().items()]
    dense = torch.randn(24, 16, 3, 3, generator=torch.Generator().manual_seed(1))
    c = T.TKConv2dC_B200(16, 24, 3, padding=1, hp_dict=HP, name="l", dense_w=dense)   # factorised at load
    w = torch.einsum("abrs,ka,bc->kcrs", c.core_kernel.data, c.last_kernel.data[:, :, 0, 0], c.first_kernel.data[:, :, 0, 0])
    assert 0 < float(torch.linalg.norm(w - dense) / torch.linalg.norm(dense)) < 0.9


def test_reference_m_variant_runs_the_chain_the_gpu_test_compares_with(built):
    """Where the reference tree is mounted (never on the GPU box): its own TKConv2dM, loaded with our module's state dict,
    gives bit for bit the F.linear / F.conv2d chain that the GPU test below uses as its reference."""
    if not ref_import.available():
        pytest.skip("reference tree not mounted")
    from tdc_b200.tkconv_variants import TKConv2dM_B200
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 16, 14, 14, generator=g)
    m = TKConv2dM_B200(16, 24, 3, stride=2, padding=1, hp_dict=HP, name="l")
    with torch.no_grad():
        m.bias.normal_(generator=g)
    F = torch.nn.functional
    ref = F.linear(x.permute(0, 2, 3, 1), m.first_factor).permute(0, 3, 1, 2)
    ref = F.conv2d(ref, m.core_kernel, None, 2, 1)
    ref = F.linear(ref.permute(0, 2, 3, 1), m.last_factor, m.bias).permute(0, 3, 1, 2).detach()
    TK = ref_import.import_tkconv()
    rm = TK.TKConv2dM(16, 24, 3, stride=2, padding=1, hp_dict=HP, name="l")
    rm.load_state_dict(m.state_dict())
    assert torch.equal(rm(x).detach(), ref)


def test_reference_network_builder_takes_our_module_as_its_conv_class(built):
    """The drop-in claim for the Python surface: the reference's own _tt_resnet(TTBasicBlock, [2,2,2,2], conv=...)
    (inference/resnet_inet_tt.py:432-448) builds with TKConv2dC_B200 injected as the conv class, and the network it
    makes has exactly the state-dict keys and shapes it has with the reference's TKConv2dC."""
    if not ref_import.available():
        pytest.skip("reference tree not mounted")
    import tdc_b200 as T
    R = ref_import.import_resnet()
    TK = ref_import.import_tkconv()
    hp = T.HalfRanks((2, 2, 2, 2))
    ours = R._tt_resnet(R.TTBasicBlock, [2, 2, 2, 2], conv=T.TKConv2dC_B200, hp_dict=hp)
    theirs = R._tt_resnet(R.TTBasicBlock, [2, 2, 2, 2], conv=TK.TKConv2dC, hp_dict=hp)
    ko = [(k, tuple(v.shape)) for k, v in ours.state_dict().items()]
    kt = [(k, tuple(v.shape)) for k, v in theirs.state_dict().items()]
    assert ko == kt and sum(isinstance(m, T.TKConv2dC_B200) for m in ours.modules()) == 16
    ours.load_state_dict(theirs.state_dict())           # a checkpoint of the reference network loads unchanged


@pytest.mark.gpu
def test_m_and_r_variants_agree_with_the_reference_chain(built):
    import tdc_b200 as T
    from tdc_b200.tkconv_variants import TKConv2dM_B200, TKConv2dR_B200
    g = torch.Generator().manual_seed(5)
    x = torch.randn(3, 16, 14, 14, generator=g)
    m = TKConv2dM_B200(16, 24, 3, stride=2, padding=1, hp_dict=HP, name="l")
    with torch.no_grad():
        m.bias.normal_(generator=g)
    # the reference TKConv2dM forward: F.linear on NHWC views around the core conv (TKConv.py:202-209)
    F = torch.nn.functional
    ref = F.linear(x.permute(0, 2, 3, 1), m.first_factor).permute(0, 3, 1, 2)
    ref = F.conv2d(ref, m.core_kernel, None, 2, 1)
    ref = F.linear(ref.permute(0, 2, 3, 1), m.last_factor, m.bias).permute(0, 3, 1, 2).detach()
    y = m.cuda()(x.cuda())
    assert rel_err(y.cpu().numpy(), ref.numpy()) <= FP32_TOL
    r = TKConv2dR_B200(16, 24, 3, stride=2, padding=1, hp_dict=HP, name="l")
    with torch.no_grad():
        r.first_factor.copy_(m.first_factor); r.core_tensor.copy_(m.core_kernel); r.last_factor.copy_(m.last_factor)
        r.bias.copy_(m.bias)
    yr = r.cuda()(x.cuda())
    assert rel_err(yr.cpu().numpy(), ref.numpy()) <= FP32_TOL        # one dense conv == the three-conv chain
