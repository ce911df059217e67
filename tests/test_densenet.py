"""TK-compressed DenseNet-121 and the SVD 1x1 convs: key compatibility with the reference (CPU) and output parity with
the reference's own TenDenseNet run on CPU (GPU; golden logits in tests/golden/tk_densenet121.npz, written by
tests/golden/make_golden_densenet121.py)."""
import os
import sys

import numpy as np
import pytest
import torch

from helpers import GOLDEN, NET_FP32_TOL, NET_TC_TOL, ROOT, rel_err

Z = np.load(os.path.join(GOLDEN, "tk_densenet121.npz"))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def test_state_dict_keys_and_ranks_match_the_reference(built):
    import tdc_b200 as T
    m = T.tkc_densenet121()
    assert sorted(m.state_dict().keys()) == list(Z["keys"])
    assert sorted(T.Growth32Ranks().ranks.keys()) == list(Z["rank_keys"])       # the reference's shipped dictionary
    layer = m.features.denseblock3.denselayer24
    assert isinstance(layer.conv2, T.TKConv2dC_B200) and tuple(layer.conv2.core_kernel.shape) == (32, 32, 3, 3)
    assert isinstance(layer.conv1, torch.nn.Conv2d) and tuple(layer.conv1.weight.shape) == (128, 256 + 23 * 32, 1, 1)
    assert tuple(m.features.transition2.conv.weight.shape) == (256, 512, 1, 1) and m.classifier.in_features == 1024
    assert sum(p.numel() for p in m.parameters()) == 6672232
    with pytest.raises(T.TdcError):
        m.train()(torch.zeros(1, 3, 64, 64))


def test_svd_branches_follow_the_rank_dictionary(built):
    import tdc_b200 as T
    from make_golden_densenet121 import small_ranks
    m = T.TKDenseNet(32, (2, 2), hp_dict=small_ranks())
    assert sorted(m.state_dict().keys()) == list(Z["small_keys"])
    c = m.features.denseblock1.denselayer2.conv1
    assert isinstance(c, T.SVDConv2dC_B200) and c.rank == 16 and tuple(c.left_kernel.shape) == (16, 96, 1, 1)
    assert tuple(c.right_kernel.shape) == (128, 16, 1, 1) and c.bias is None
    assert isinstance(m.features.transition1.conv, T.SVDConv2dC_B200)
    assert isinstance(m.features.denseblock2.denselayer1.conv1, torch.nn.Conv2d)


def test_svd_conv_constructor_contract(built):
    """The reference's checks (SVDConv.py:135-142) and its initialisation from a dense weight (:175-181): the two
    factors multiply to the best rank-r approximation."""
    import tdc_b200 as T

    class HP:
        ranks = {"a": [8], "b": 5}
    for cls in (T.SVDConv2dC_B200, T.SVDConv2dM_B200, T.SVDConv2dR_B200):
        with pytest.raises(ValueError):
            cls(16, 24, 3, hp_dict=HP, name="a")
        with pytest.raises(ValueError):
            cls(16, 24, 1, stride=2, hp_dict=HP, name="a")
        with pytest.raises(ValueError):
            cls(16, 24, 1, groups=2, hp_dict=HP, name="a")
        assert cls(16, 24, 1, hp_dict=HP, name="b").rank == 5
    g = torch.Generator().manual_seed(3)
    w = torch.randn(24, 16, 1, 1, generator=g)
    m = T.SVDConv2dC_B200(16, 24, 1, bias=True, hp_dict=HP, name="a", dense_w=w, dense_b=torch.arange(24.0))
    u, s, vt = np.linalg.svd(w.squeeze().numpy().astype(np.float64), full_matrices=False)
    best = (u[:, :8] * s[:8]) @ vt[:8]
    got = m.right_kernel.detach().squeeze().double().numpy() @ m.left_kernel.detach().squeeze().double().numpy()
    assert np.abs(got - best).max() <= 1e-6 and float(m.bias.detach()[3]) == 3.0
    r = T.SVDConv2dR_B200(16, 24, 1, hp_dict=HP, name="a", dense_w=w)
    assert tuple(r.left_factor.shape) == (8, 16) and tuple(r.right_factor.shape) == (24, 8)
    assert np.abs(r._recover_weight().detach().squeeze().double().numpy() - best).max() <= 1e-6
    full = T.SVDConv2dC_B200(16, 24, 1, bias=False, hp_dict=type("H", (), {"ranks": {"a": [16]}}), name="a", dense_w=w)
    got = full.right_kernel.detach().squeeze() @ full.left_kernel.detach().squeeze()
    assert float((got - w.squeeze()).abs().max()) <= 1e-5          # full rank reproduces the dense weight


def test_svd_conv_state_dict_loads_from_the_reference_class(built):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_import
    if not ref_import.available():
        pytest.skip("reference tree not mounted")
    import tdc_b200 as T
    S = ref_import.import_svdconv()

    class HP:
        ranks = {"a": [8]}
    g = torch.Generator().manual_seed(5)
    w = torch.randn(24, 16, 1, 1, generator=g)
    ref = S.SVDConv2dC(16, 24, 1, hp_dict=HP, name="a", bias=True)
    mine = T.SVDConv2dC_B200(16, 24, 1, hp_dict=HP, name="a", bias=True)
    assert {k: tuple(v.shape) for k, v in ref.state_dict().items()} == {k: tuple(v.shape) for k, v in mine.state_dict().items()}
    mine.load_state_dict(ref.state_dict())
    # the reference's SVDConv2dR multiplies its factors in the order left @ right ([r,C] x [K,r]) when it recovers
    # the weight, so it cannot be built unless C == K == r; parameter names and shapes are taken from its constructor
    with pytest.raises(RuntimeError):
        S.SVDConv2dR(16, 24, 1, hp_dict=HP, name="a", bias=True)
    sq = S.SVDConv2dR(8, 8, 1, hp_dict=HP, name="a", bias=True)
    mine_r = T.SVDConv2dR_B200(8, 8, 1, hp_dict=HP, name="a", bias=True)
    assert {k: tuple(v.shape) for k, v in sq.state_dict().items()} == {k: tuple(v.shape) for k, v in mine_r.state_dict().items()}
    # the SVD initialisation spans the same rank-8 subspace as the reference's numpy SVD
    ref = S.SVDConv2dC(16, 24, 1, hp_dict=HP, name="a", bias=False, dense_w=w)
    mine = T.SVDConv2dC_B200(16, 24, 1, hp_dict=HP, name="a", bias=False, dense_w=w)
    a = ref.right_kernel.detach().squeeze() @ ref.left_kernel.detach().squeeze()
    b = mine.right_kernel.detach().squeeze() @ mine.left_kernel.detach().squeeze()
    assert float((a - b).abs().max()) <= 1e-5
    x = torch.randn(2, 16, 5, 5, generator=g)
    assert ref(x).shape == (2, 24, 5, 5)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(2, 40, 14, 14, 72), (1, 24, 7, 7, 24), (3, 16, 5, 6, 48), (2, 8, 56, 56, 8)])
def test_affine_relu_on_channel_slices(built, shape):
    """Scale/shift/ReLU reading a channel prefix of a larger buffer, and the strided copy that appends features."""
    import tdc_b200 as T
    B, C, H, W, Ctot = shape
    g = torch.Generator().manual_seed(sum(shape))
    buf = torch.randn(B, Ctot, H, W, generator=g).cuda()
    scale, shift = (torch.rand(C, generator=g) + 0.5).cuda(), torch.randn(C, generator=g).cuda()
    y = T.affine_relu(buf[:, :C], scale, shift, relu=True)
    ref = torch.relu(buf[:, :C] * scale.view(1, -1, 1, 1) + shift.view(1, -1, 1, 1))
    assert y.is_contiguous() and float((y - ref).abs().max()) <= 1e-6
    y2 = T.affine_relu(buf[:, :C], scale, None, relu=False)
    assert torch.equal(y2, buf[:, :C] * scale.view(1, -1, 1, 1))
    before = buf.clone()
    T.affine_relu(y, None, None, relu=False, out=buf[:, Ctot - C:])
    assert torch.equal(buf[:, Ctot - C:], y) and torch.equal(buf[:, :Ctot - C], before[:, :Ctot - C])
    with pytest.raises(T.TdcError):
        T.affine_relu(buf[:, :, ::2], scale, shift)
    with pytest.raises(T.TdcError):
        T.affine_relu(buf[:, :C], scale, shift, out=torch.empty(B, C + 1, H, W, device="cuda"))


@pytest.mark.gpu
@pytest.mark.parametrize("cls_name", ["SVDConv2dC_B200", "SVDConv2dM_B200", "SVDConv2dR_B200"])
@pytest.mark.parametrize("precision", ["fp32", "tf32x3"])
def test_svd_conv_forward(built, cls_name, precision):
    """Two chained 1x1 convs + bias, against the same chain in fp64 (SVDConv2dC.forward, SVDConv.py:190-194)."""
    import tdc_b200 as T

    class HP:
        ranks = {"a": [24]}
    g = torch.Generator().manual_seed(11)
    m = getattr(T, cls_name)(96, 64, 1, bias=True, hp_dict=HP, name="a").cuda()
    m.precision = precision
    with torch.no_grad():
        m.bias.copy_(torch.randn(64, generator=g))
    x = torch.randn(4, 96, 28, 28, generator=g).cuda()
    left, right = m._kernels()
    ref = torch.nn.functional.conv2d(torch.nn.functional.conv2d(x.double(), left.detach().double()), right.detach().double(), m.bias.detach().double())
    with torch.no_grad():
        y = m(x)
    assert rel_err(y.cpu().numpy(), ref.cpu().numpy()) <= 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("precision", ["fp32", "auto"])
def test_logits_match_the_reference_network(built, precision):
    import tdc_b200 as T
    m = T.fill_deterministic(T.tkc_densenet121(precision=precision).eval(), seed=0, gain=0.7).cuda()
    x = torch.randn(2, 3, 112, 112, generator=torch.Generator().manual_seed(121)).cuda()
    feats = {}
    m.features.denseblock1.register_forward_hook(lambda mod, i, o: feats.__setitem__("block1", o))
    with torch.no_grad():
        final = m.forward_features(x)
        logits = m(x)
    # 120 chained convolutions with BatchNorm between them: the fp32 kernels at the single-layer bar, the tensor-core
    # tier at its own
    tol = NET_FP32_TOL if precision == "fp32" else NET_TC_TOL
    assert rel_err(feats["block1"][0].mean((1, 2)).cpu().numpy(), Z["block1_mean"]) <= tol
    assert rel_err(final[0].mean((1, 2)).cpu().numpy(), Z["final_mean"]) <= tol
    assert rel_err(logits.cpu().numpy(), Z["logits"]) <= tol
    assert (logits.argmax(1).cpu().numpy() == Z["logits"].argmax(1)).all()


@pytest.mark.gpu
@pytest.mark.parametrize("precision", ["fp32", "tf32x3"])
def test_network_with_svd_convs_matches_the_reference(built, precision):
    import tdc_b200 as T
    from make_golden_densenet121 import small_ranks
    m = T.fill_deterministic(T.TKDenseNet(32, (2, 2), hp_dict=small_ranks(), precision=precision).eval(), seed=1).cuda()
    x = torch.randn(3, 3, 64, 64, generator=torch.Generator().manual_seed(122)).cuda()
    with torch.no_grad():
        logits = m(x)
    assert rel_err(logits.cpu().numpy(), Z["small_logits"]) <= 2e-5


@pytest.mark.gpu
def test_graphed_forward_replays_the_eager_result(built):
    """A forward captured as a CUDA graph gives the eager forward's bits, for new inputs too."""
    import tdc_b200 as T
    m = T.fill_deterministic(T.TKDenseNet(32, (2, 2)).eval(), seed=2, gain=0.7).cuda()
    g = torch.Generator().manual_seed(7)
    x0, x1 = torch.randn(1, 3, 64, 64, generator=g).cuda(), torch.randn(1, 3, 64, 64, generator=g).cuda()
    graphed = T.GraphedForward(m, x0)
    with torch.no_grad():
        assert torch.equal(graphed(x1).clone(), m(x1)) and torch.equal(graphed(x0).clone(), m(x0))
    with pytest.raises(ValueError):
        graphed(torch.zeros(2, 3, 64, 64, device="cuda"))
    r = T.fill_deterministic(T.tkc_resnet18(precision="auto").eval(), seed=0).cuda()
    x = torch.randn(1, 3, 224, 224, generator=g).cuda()
    gr = T.GraphedForward(r, x)
    with torch.no_grad():
        assert torch.equal(gr(x).clone(), r(x))
