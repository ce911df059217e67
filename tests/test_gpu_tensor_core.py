"""The tensor-core variant (tcgen05, TF32 or fp16 operands) against the fp64 arbiter, through the C ABI.
modes 3 and 4 (operands split into two TF32 / two fp16 parts) are held to the fp32 bar of 1e-5 per layer;
mode 1 (plain TF32) to 5e-3."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from helpers import FP32_TOL, NET_TC_TOL, SWEEP, draw_core, rel_err

TF32_TOL = 5e-3


@pytest.fixture(scope="module")
def T(built):
    import tdc_b200
    return tdc_b200


def test_plan_is_made_on_the_host(T):
    from tdc_b200 import _lib
    p = _lib.TcPlan()
    assert T.lib.tdc_tc_plan_make(64, 64, 3, 3, 3, C.byref(p)) == 0
    assert (p.nt, p.cb, p.nkb, p.n_ocb, p.hl) == (64, 8, 8, 1, 2) and p.weights_bytes == 4 * 2 * 9 * 8 * 64 * 8
    assert T.lib.tdc_tc_plan_make(20, 200, 1, 1, 1, C.byref(p)) == 0
    assert (p.nt, p.nkb, p.n_ocb, p.hl) == (128, 3, 2, 1)
    assert T.lib.tdc_tc_plan_make(64, 64, 5, 5, 3, C.byref(p)) == _lib.ERR_UNSUPPORTED
    assert T.lib.tdc_tc_plan_make_general(3, 64, 7, 7, 3, C.byref(p)) == 0          # the stem: 147 "channels" in 19 blocks of 8
    assert (p.general, p.nt, p.nkb, p.n_ocb, p.hl) == (1, 64, 19, 1, 2) and p.weights_bytes == 4 * 2 * 1 * 8 * 64 * 19
    assert T.lib.tdc_tc_plan_make_general(3, 64, 0, 7, 3, C.byref(p)) == _lib.ERR_SHAPE
    assert T.lib.tdc_tc_plan_make(64, 64, 3, 3, 4, C.byref(p)) == 0                   # fp16 parts: 16 channels per K step, a scratch tail
    assert (p.nt, p.cb, p.nkb, p.n_ocb, p.hl) == (64, 16, 4, 1, 2) and p.weights_bytes == 4 * 2 * 9 * 8 * 64 * 4 + 4 * (1024 + 64)
    assert T.lib.tdc_tc_plan_make(64, 64, 3, 3, 2, C.byref(p)) == _lib.ERR_UNSUPPORTED
    # strided rows: the stem gathers 3 channels x 7 filter rows x 2 column phases = 42 values in 3 blocks of 16 and takes
    # the 4 column steps as taps; a 3x3 stride-2 core gathers 6 per channel and takes 2 taps
    assert T.lib.tdc_tc_plan_make_strided(3, 64, 7, 7, 2, 3, 4, 0, C.byref(p)) == 0
    assert (p.general, p.stride, p.phase, p.nt, p.cb, p.nkb) == (2, 2, 1, 64, 16, 3) and p.weights_bytes == 4 * 2 * 4 * 8 * 64 * 3 + 4 * (1024 + 64)
    assert T.lib.tdc_tc_plan_make_strided(64, 128, 3, 3, 2, 1, 4, 0, C.byref(p)) == 0
    assert (p.general, p.stride, p.phase, p.nt, p.nkb) == (2, 2, 1, 128, 24) and p.weights_bytes == 4 * 2 * 2 * 8 * 128 * 24 + 4 * (1024 + 64)
    # an even padding needs no phase; a 4-wide filter keeps its 2 taps only without one; other strides have none
    assert T.lib.tdc_tc_plan_make_strided(64, 128, 3, 3, 2, 0, 4, 0, C.byref(p)) == 0 and p.phase == 0
    assert T.lib.tdc_tc_plan_make_strided(8, 8, 4, 4, 2, 1, 4, 0, C.byref(p)) == 0 and p.phase == 0
    assert T.lib.tdc_tc_plan_make_strided(8, 8, 3, 7, 4, 1, 4, 0, C.byref(p)) == 0 and p.phase == 0
    assert T.lib.tdc_tc_plan_make_strided(8, 8, 5, 5, 2, 2, 4, 0, C.byref(p)) == _lib.ERR_UNSUPPORTED      # 3 column steps
    assert T.lib.tdc_tc_plan_make_strided(8, 8, 3, 3, 2, 1, 3, 0, C.byref(p)) == _lib.ERR_UNSUPPORTED      # fp16 parts only
    assert T.lib.tdc_tc_plan_make(0, 64, 3, 3, 3, C.byref(p)) == _lib.ERR_SHAPE
    assert b"mode" in T.lib.tdc_tc_last_error_string() or b"C=" in T.lib.tdc_tc_last_error_string()


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,K,H,W,R", [(1, 8, 32, 8, 8, 1), (2, 16, 32, 12, 12, 3), (3, 20, 40, 7, 7, 3), (2, 32, 96, 14, 14, 1),
                                           (5, 33, 130, 9, 13, 3), (1, 3, 5, 1, 1, 1), (2, 7, 9, 2, 3, 3), (1, 128, 128, 28, 28, 3),
                                           (4, 64, 64, 56, 56, 3), (2, 24, 16, 5, 200, 3)])
def test_against_arbiter(T, B, Cc, K, H, W, R):
    from tdc_b200 import tc
    x, w = draw_core(700 + B + Cc + H, B, Cc, K, H, W, R)
    ref = O.conv2d_f64(x.numpy(), w.numpy(), pad=(R - 1) // 2)
    for mode, tol in ((4, FP32_TOL), (1, TF32_TOL), (3, FP32_TOL)):
        y = T.TcConv(w.cuda(), mode=mode)(x.cuda()).cpu().numpy()
        assert y.shape == ref.shape and rel_err(y, ref) <= tol, (mode, rel_err(y, ref))
    crsk = np.ascontiguousarray(w.numpy().transpose(1, 2, 3, 0))
    for mode in (3, 4):          # the channel-last filter layout prepares the same operands: every bit agrees
        y2 = T.TcConv(torch.from_numpy(crsk).cuda(), mode=mode, w_layout=T.W_CRSK)(x.cuda()).cpu().numpy()
        assert rel_err(y2, ref) <= FP32_TOL and (mode != 3 or np.array_equal(y2, y))
    assert tc.status() == 0          # no bounded wait ran out


@pytest.mark.gpu
@pytest.mark.parametrize("H,R1,R2", SWEEP)
def test_sweep_shapes_meet_the_fp32_bar(T, H, R1, R2):
    """Batch 64 of every sweep shape: four sampled images against the arbiter; integer inputs
    with all-ones weights exactly (the reference drivers' own check)."""
    i = SWEEP.index((H, R1, R2))
    x, w = draw_core(2100 + i, 64, R1, R2, H, H)
    sel = [0, 21, 42, 63]
    ref = O.conv2d_f64(x[sel].numpy(), w.numpy(), pad=1)
    xi = torch.randint(0, 10, (2, R1, H, H), generator=torch.Generator().manual_seed(i)).float()
    ones = torch.ones(R2, R1, 3, 3)
    for mode in (3, 4):
        y = T.TcConv(w.cuda(), mode=mode)(x.cuda())
        assert rel_err(y[sel].cpu().numpy(), ref) <= FP32_TOL, mode
        yi = T.TcConv(ones.cuda(), mode=mode)(xi.cuda()).cpu().numpy()
        assert np.array_equal(yi, O.conv2d_f64(xi.numpy(), ones.numpy(), pad=1)), mode
    # the fp16 mode is the closer of the two to fp64: half as many accumulations feed each running sum
    assert rel_err(y[sel].cpu().numpy(), ref) <= 4e-6


@pytest.mark.gpu
def test_epilogue_and_errors(T):
    g = torch.Generator().manual_seed(9)
    x = torch.randn(3, 16, 14, 14, generator=g).cuda()
    w = (torch.randn(24, 16, 3, 3, generator=g) * 0.1).cuda()
    scale, shift = (torch.rand(24, generator=g) + 0.5).cuda(), torch.randn(24, generator=g).cuda()
    res = torch.randn(3, 24, 14, 14, generator=g).cuda()
    ref = torch.relu(torch.nn.functional.conv2d(x.double(), w.double(), padding=1) * scale.double().view(1, -1, 1, 1)
                     + shift.double().view(1, -1, 1, 1) + res.double())
    for mode in (3, 4):
        y = T.TcConv(w, mode=mode)(x, scale, shift, res, True)
        assert rel_err(y.cpu().numpy(), ref.cpu().numpy()) <= FP32_TOL
    with pytest.raises(T.TdcError):
        T.TcConv(torch.zeros(4, 4, 5, 5).cuda())
    with pytest.raises(T.TdcError):
        T.TcConv(w)(torch.zeros(1, 8, 4, 4).cuda())


@pytest.mark.gpu
def test_module_and_network_precisions(T):
    class HP:
        ranks = {"l": [24, 16]}
    torch.manual_seed(3)
    m = T.TKConv2dC_B200(32, 48, 3, stride=1, padding=1, bias=True, hp_dict=HP, name="l").cuda()
    x = torch.randn(4, 32, 28, 28).cuda()
    with torch.no_grad():
        y32 = m(x)
        m.precision = "tf32x3"
        y3 = m(x)
        m.precision = "fp16x3"
        y4 = m(x)
        m.precision = "tf32"
        y1 = m(x)
    assert rel_err(y3.cpu().numpy(), y32.cpu().numpy()) <= FP32_TOL and rel_err(y4.cpu().numpy(), y32.cpu().numpy()) <= FP32_TOL
    assert FP32_TOL < rel_err(y1.cpu().numpy(), y32.cpu().numpy()) <= TF32_TOL
    net = T.fill_deterministic(T.tkc_resnet18().eval(), 0).cuda()
    xin = torch.randn(8, 3, 224, 224, generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        a = net(xin)
        b = net.set_precision("auto")(xin)
    assert rel_err(b.cpu().numpy(), a.cpu().numpy()) <= NET_TC_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,K,H,W,R", [(1, 3, 5, 1, 1, 1), (2, 7, 9, 2, 3, 3), (5, 33, 130, 9, 13, 3), (70, 24, 40, 14, 14, 3),
                                           (9, 64, 64, 56, 56, 3), (300, 16, 32, 7, 7, 3), (33, 40, 64, 15, 15, 1), (16, 32, 32, 28, 28, 1),
                                           (100, 24, 128, 28, 28, 3), (47, 16, 64, 56, 56, 1)])
def test_persistent_and_one_tile_kernels_agree(T, B, Cc, K, H, W, R, monkeypatch):
    """The launcher has two kernels (one tile per CTA; persistent CTAs walking a tile list with the accumulators
    handed over tile by tile).  Both are forced in turn through the environment switch the launcher reads per call,
    with and without the fused epilogue, on shapes with fewer tiles than SMs, several tiles per CTA, ragged channel
    counts and one-pixel images: same arithmetic in the same order, so the outputs must be bit-identical, and the
    persistent one is checked against the fp64 arbiter on sampled images."""
    from tdc_b200 import tc
    x, w = draw_core(900 + B + Cc + H, B, Cc, K, H, W, R)
    g = torch.Generator().manual_seed(B + K)
    scale, shift = (torch.rand(K, generator=g) + 0.5).cuda(), torch.randn(K, generator=g).cuda()
    res = torch.randn(B, K, H, W, generator=g).cuda()
    xd, wd = x.cuda(), w.cuda()
    sel = sorted({0, B // 2, B - 1})
    ref = O.conv2d_f64(x[sel].numpy(), w.numpy(), pad=(R - 1) // 2)
    for mode, tol in ((3, FP32_TOL), (1, TF32_TOL)):
        conv = T.TcConv(wd, mode=mode)
        out = {}
        for persist in ("0", "1"):
            monkeypatch.setenv("TDC_TC_PERSIST", persist)
            out[persist] = (conv(xd).clone(), conv(xd, scale, shift, res, True).clone())
        assert torch.equal(out["0"][0], out["1"][0]) and torch.equal(out["0"][1], out["1"][1]), mode
        assert rel_err(out["1"][0][sel].cpu().numpy(), ref) <= tol
        want = np.maximum(ref * scale.cpu().numpy()[None, :, None, None] + shift.cpu().numpy()[None, :, None, None] + res[sel].cpu().numpy(), 0)
        assert rel_err(out["1"][1][sel].cpu().numpy(), want) <= tol
        if mode == 3:
            y3 = out["1"][0]
    for knobs in ({"TDC_TC_MT": "1"}, {"TDC_TC_MT": "2", "TDC_TC_NBUF": "1"}, {"TDC_TC_NS": "2", "TDC_TC_DEPTH": "2"}, {"TDC_TC_TAIL": "0"}, {"TDC_TC_KPS": "1"},
                  {"TDC_TC_VEC": "0"}, {"TDC_TC_VEC": "1"}):
        for k, v in knobs.items():
            monkeypatch.setenv(k, v)
        assert torch.equal(T.TcConv(wd, mode=3)(xd), y3), knobs      # tile count, buffers and ring depth change no bit
        for k in knobs:
            monkeypatch.delenv(k)
    assert tc.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,K,H,W", [(128, 64, 128, 56, 56), (64, 32, 64, 56, 56), (32, 224, 128, 28, 28), (32, 256, 128, 14, 14),
                                         (40, 96, 32, 28, 28), (3, 520, 256, 12, 12)])
def test_one_tap_loaders_agree(T, B, Cc, K, H, W, monkeypatch):
    """A 1x1 filter on images of a multiple of 4 pixels can be staged by 16-byte loads or through the cp.async ring;
    the launcher picks by layer size.  Both forced in turn, in the persistent kernel with and without the smaller
    tiles of the last round and in the one-tile kernel: the operands are the same values in the same places, so every
    output bit agrees, and the first and last images are checked against fp64."""
    from tdc_b200 import tc
    g = torch.Generator().manual_seed(B + Cc + K)
    x = torch.randn(B, Cc, H, W, generator=g).cuda()
    w = (torch.randn(K, Cc, 1, 1, generator=g) * 0.1).cuda()
    conv = T.TcConv(w, mode=3)
    y = conv(x).clone()
    for knobs in ({"TDC_TC_VEC": "0"}, {"TDC_TC_VEC": "1"}, {"TDC_TC_VEC": "0", "TDC_TC_TAIL": "0"}, {"TDC_TC_VEC": "0", "TDC_TC_PERSIST": "1"},
                  {"TDC_TC_VEC": "1", "TDC_TC_PERSIST": "1"}, {"TDC_TC_VEC": "0", "TDC_TC_PERSIST": "0"}, {"TDC_TC_VEC": "0", "TDC_TC_MT": "1"}):
        for k, v in knobs.items():
            monkeypatch.setenv(k, v)
        assert torch.equal(conv(x), y), knobs
        for k in knobs:
            monkeypatch.delenv(k)
    for sel in (slice(0, 2), slice(B - 2, B)):
        ref = torch.nn.functional.conv2d(x[sel].double(), w.double())
        assert float((y[sel].double() - ref).abs().max() / ref.abs().max()) <= FP32_TOL
    assert tc.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,K,H,W,stride", [(4, 64, 128, 56, 56, 2), (3, 24, 40, 15, 13, 2), (2, 16, 32, 9, 9, 3), (70, 128, 256, 28, 28, 2)])
def test_strided_1x1_shortcut(T, B, Cc, K, H, W, stride, monkeypatch):
    """The down-sampling shortcut of a residual stage (a 1x1 filter with a stride): both kernels, both modes,
    with the folded-BatchNorm epilogue, against the fp64 arbiter."""
    from tdc_b200 import tc
    x, w = draw_core(1300 + B + Cc + H, B, Cc, K, H, W, 1)
    g = torch.Generator().manual_seed(K)
    scale, shift = (torch.rand(K, generator=g) + 0.5).cuda(), torch.randn(K, generator=g).cuda()
    sel = sorted({0, B // 2, B - 1})
    ref = O.conv2d_f64(x[sel].numpy(), w.numpy(), pad=0, stride=stride)
    want = ref * scale.cpu().numpy()[None, :, None, None] + shift.cpu().numpy()[None, :, None, None]
    assert tc.supported(1, 1, stride, 0, W) and not tc.supported(3, 3, stride, 1, W)
    for mode, tol in ((3, FP32_TOL), (1, TF32_TOL), (4, FP32_TOL)):
        conv = T.TcConv(w.cuda(), mode=mode)
        for persist in ("0", "1"):
            monkeypatch.setenv("TDC_TC_PERSIST", persist)
            y = conv(x.cuda(), scale, shift, stride=stride)
            assert tuple(y.shape) == (B, K, (H - 1) // stride + 1, (W - 1) // stride + 1)
            assert rel_err(y[sel].cpu().numpy(), want) <= tol, (mode, persist)
    with pytest.raises(T.TdcError):
        T.TcConv(torch.zeros(8, 8, 3, 3).cuda())(x.cuda()[:, :8], stride=2)
    assert tc.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,K,H,W,R,stride,pad", [(2, 3, 64, 32, 32, 7, 2, 3), (3, 16, 24, 15, 13, 3, 2, 1), (2, 8, 16, 9, 9, 5, 1, 2),
                                                      (1, 4, 8, 6, 7, 3, 3, 0), (40, 64, 64, 28, 28, 3, 2, 1), (3, 5, 130, 8, 8, 3, 1, 1),
                                                      (2, 32, 32, 12, 12, 1, 1, 0)])
def test_general_plan(T, B, Cc, K, H, W, R, stride, pad):
    """The gathering plan (any filter size, stride, padding; the stem and the strided cores of the residual
    networks): both modes and both filter layouts against the fp64 arbiter, and bit-identical to the
    one-pass plan where that one applies (the same products summed in a different channel order would not be;
    here the order is the same only for 1x1 filters)."""
    from tdc_b200 import tc
    x, w = draw_core(1700 + B + Cc + H + R, B, Cc, K, H, W, R)
    sel = sorted({0, B // 2, B - 1})
    ref = O.conv2d_f64(x[sel].numpy(), w.numpy(), pad=pad, stride=stride)
    g = torch.Generator().manual_seed(K + R)
    scale, shift = (torch.rand(K, generator=g) + 0.5).cuda(), torch.randn(K, generator=g).cuda()
    for mode, tol in ((3, FP32_TOL), (1, TF32_TOL), (4, FP32_TOL)):
        conv = T.TcConv(w.cuda(), mode=mode, general=True)
        y = conv(x.cuda(), stride=stride, padding=pad)
        assert tuple(y.shape[1:]) == ref.shape[1:] and rel_err(y[sel].cpu().numpy(), ref) <= tol, (mode, rel_err(y[sel].cpu().numpy(), ref))
        y = conv(x.cuda(), scale, shift, None, True, stride=stride, padding=pad)
        want = np.maximum(ref * scale.cpu().numpy()[None, :, None, None] + shift.cpu().numpy()[None, :, None, None], 0)
        assert rel_err(y[sel].cpu().numpy(), want) <= tol
    crsk = torch.from_numpy(np.ascontiguousarray(w.numpy().transpose(1, 2, 3, 0))).cuda()
    y2 = T.TcConv(crsk, mode=3, w_layout=T.W_CRSK, general=True)(x.cuda(), stride=stride, padding=pad)
    assert torch.equal(y2, T.TcConv(w.cuda(), mode=3, general=True)(x.cuda(), stride=stride, padding=pad))
    if R == 1:
        assert torch.equal(y2, T.TcConv(w.cuda(), mode=3)(x.cuda(), stride=stride))
    assert tc.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,K,H,W,R,S,stride,pad", [(2, 3, 64, 38, 38, 7, 7, 2, 3), (3, 16, 24, 15, 13, 3, 3, 2, 1), (70, 32, 48, 14, 14, 3, 3, 2, 1),
                                                        (2, 5, 9, 11, 17, 4, 4, 2, 0), (1, 7, 130, 9, 9, 8, 8, 2, 3), (2, 6, 8, 21, 20, 3, 7, 4, 2),
                                                        (3, 33, 40, 10, 12, 2, 4, 3, 1), (300, 8, 16, 5, 5, 3, 3, 2, 1), (2, 64, 64, 56, 56, 3, 3, 2, 1),
                                                        (3, 9, 20, 12, 14, 3, 3, 2, 0), (2, 6, 10, 16, 18, 7, 7, 2, 2), (5, 12, 16, 9, 11, 3, 3, 2, 1),
                                                        (2, 4, 8, 10, 10, 7, 3, 2, 1)])
def test_strided_row_plan(T, B, Cc, K, H, W, R, S, stride, pad):
    """The plan for strided layers with 2 or 4 column steps (stem 7x7 / 2, cores 3x3 / 2): the contraction runs over
    (channel, filter row, column phase) and the column steps are MMA taps one output position apart.  Against the fp64
    arbiter with and without the epilogue, both filter layouts bit-identical, odd images, filters wider than tall,
    strides 2 to 4, batches that put many images in one tile and spread them over many CTAs."""
    from tdc_b200 import tc
    assert tc.strided_rows(S, stride)
    g = torch.Generator().manual_seed(2900 + B + Cc + H + S)
    x = torch.randn(B, Cc, H, W, generator=g)
    w = torch.randn(K, Cc, R, S, generator=g) * (2.0 / (Cc * R * S)) ** 0.5
    sel = sorted({0, B // 2, B - 1})
    ref = torch.nn.functional.conv2d(x[sel].double(), w.double(), None, stride, pad).numpy()
    conv = T.TcConv(w.cuda(), mode=4, general=True)
    y = conv(x.cuda(), stride=stride, padding=pad)
    assert tuple(y.shape[1:]) == ref.shape[1:] and rel_err(y[sel].cpu().numpy(), ref) <= FP32_TOL, rel_err(y[sel].cpu().numpy(), ref)
    assert any(k[1] == (stride, pad & 1) for k in conv._by_nt), "the strided-row plan did not run"
    scale, shift = (torch.rand(K, generator=g) + 0.5), torch.randn(K, generator=g)
    res = torch.randn(y.shape, generator=g)
    y2 = conv(x.cuda(), scale.cuda(), shift.cuda(), res.cuda(), True, stride=stride, padding=pad)
    want = np.maximum(ref * scale.numpy()[None, :, None, None] + shift.numpy()[None, :, None, None] + res[sel].numpy(), 0)
    assert rel_err(y2[sel].cpu().numpy(), want) <= FP32_TOL
    crsk = torch.from_numpy(np.ascontiguousarray(w.numpy().transpose(1, 2, 3, 0))).cuda()
    assert torch.equal(y, T.TcConv(crsk, mode=4, w_layout=T.W_CRSK, general=True)(x.cuda(), stride=stride, padding=pad))
    # an input that starts 4 bytes off a 16-byte boundary takes the 4-byte copies instead of the 8-byte pairs: the same values
    # through the same arithmetic, so every bit agrees
    off = torch.empty(x.numel() + 1, device="cuda")
    xv = off[1:].view(x.shape)
    xv.copy_(x)
    assert xv.data_ptr() % 16 != 0 and torch.equal(y, conv(xv, stride=stride, padding=pad))
    assert tc.status() == 0


@pytest.mark.gpu
def test_dependent_launches_wait_for_their_input(T, monkeypatch):
    """The persistent kernel is launched so that it may be scheduled while the kernel before it still runs (programmatic
    dependent launch) and waits inside for that kernel's results.  A chain in which every launch reads what the one before
    wrote — on one stream, with no host synchronisation, also as a CUDA graph, also through a buffer that is written,
    read and overwritten in turn — must give the bits of the same chain run with a synchronisation after every launch
    and of the chain without early scheduling."""
    from tdc_b200 import tc
    g = torch.Generator().manual_seed(77)
    x = torch.randn(16, 64, 28, 28, generator=g).cuda()
    convs = [T.TcConv((torch.randn(64, 64, 3, 3, generator=g) * (2.0 / (64 * 9)) ** 0.5).cuda(), mode=4) for _ in range(3)]
    bufs = [torch.empty_like(x), torch.empty_like(x)]

    def chain(sync):
        t = x
        for i in range(9):
            t = convs[i % 3](t, relu=True, out=bufs[i & 1])          # ping-pong: launch i+1 overwrites what launch i read
            if sync:
                torch.cuda.synchronize()
        return t.clone()
    want = chain(True)
    assert torch.isfinite(want).all() and float(want.abs().max()) > 0
    for _ in range(3):
        assert torch.equal(chain(False), want)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain(False)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = chain(False)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    monkeypatch.setenv("TDC_TC_PDL", "0")
    assert torch.equal(chain(False), want)
    assert tc.status() == 0


@pytest.mark.gpu
def test_random_shapes_against_fp64(T):
    """Sixty seeded random layers (ragged channel counts, tiny and odd images, batch sizes around the tile and SM
    counts, one-pass and gathering plans, random epilogue options) against the same convolution in fp64 on the GPU:
    the launcher's choices (kernel, tiles per CTA, channels per block, blocks per stage) must never change a result
    beyond the split-operand bar."""
    import random
    from tdc_b200 import tc
    F = torch.nn.functional
    rnd = random.Random(20231)
    worst = 0.0
    for case in range(60):
        general = rnd.random() < 0.35
        R = rnd.choice((1, 3, 5, 7)) if general else rnd.choice((1, 3))
        stride = rnd.choice((1, 2, 3)) if (general or R == 1) else 1
        pad = rnd.randint(0, R // 2 + 1) if general else (R - 1) // 2
        Cc, K = rnd.choice((1, 3, 8, 20, 33, 64, 72, 130)), rnd.choice((1, 5, 32, 40, 64, 96, 130, 200))
        H, W = rnd.choice((1, 2, 7, 9, 14, 28, 31)), rnd.choice((1, 3, 7, 12, 14, 28, 40))
        if H + 2 * pad < R or W + 2 * pad < R:
            continue
        B = rnd.choice((1, 2, 5, 37, 150))
        if B * Cc * H * W > 6e6 or B * K * H * W > 6e6:
            B = 2
        g = torch.Generator().manual_seed(case)
        x = torch.randn(B, Cc, H, W, generator=g).cuda()
        w = (torch.randn(K, Cc, R, R, generator=g) * (2.0 / (K * R * R)) ** 0.5).cuda()
        scale = (torch.rand(K, generator=g) + 0.5).cuda() if rnd.random() < 0.5 else None
        shift = torch.randn(K, generator=g).cuda() if rnd.random() < 0.5 else None
        relu = rnd.random() < 0.5
        ref = F.conv2d(x.double(), w.double(), None, stride, pad)
        res = torch.randn(ref.shape, generator=g).cuda() if rnd.random() < 0.4 else None
        if scale is not None:
            ref = ref * scale.double().view(1, -1, 1, 1)
        if shift is not None:
            ref = ref + shift.double().view(1, -1, 1, 1)
        if res is not None:
            ref = ref + res.double()
        if relu:
            ref = ref.relu()
        conv = T.TcConv(w, mode=3 if case % 2 else 4, general=general)
        y = conv(x, scale, shift, res, relu, stride=stride, padding=pad if general else None)
        assert y.shape == ref.shape, (case, y.shape, ref.shape)
        err = float((y.double() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        worst = max(worst, err)
        assert err <= FP32_TOL, (case, general, B, Cc, K, H, W, R, stride, pad, err)
    assert tc.status() == 0 and worst > 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("Cc,H,R,general", [(64, 56, 3, False), (256, 14, 3, False), (1024, 7, 3, False), (1024, 7, 1, False), (256, 14, 3, True)])
def test_unbiased_sums(T, Cc, H, R, general):
    """The tensor core truncates its running sum toward zero: raw sums come out too small by about 1.6e-8 per
    accumulation (the slope of error against exact value).  TDC_TC_UNBIASED puts the expected loss back: the slope
    drops under a third of the raw one (and under 7e-7), the largest and the rms error fall too; without the flag sums of
    small integers stay exact (the reference drivers' check), with it they are within the fp32 bar."""
    g = torch.Generator().manual_seed(40 + Cc)
    x = torch.randn(4, Cc, H, H, generator=g).relu().cuda()
    w = (torch.randn(Cc, Cc, R, R, generator=g) * (2.0 / (Cc * R * R)) ** 0.5).cuda()
    kw = dict(stride=2, padding=1) if general else {}
    ref = torch.nn.functional.conv2d(x.double(), w.double(), None, 2 if general else 1, 1 if general else (R - 1) // 2).flatten()
    for mode in (4, 3):
        stats = []
        for unbiased in (False, True):
            e = T.TcConv(w, mode=mode, general=general, unbiased=unbiased)(x, **kw).double().flatten() - ref
            stats.append((float((e * ref).sum() / (ref * ref).sum()), float(e.abs().max() / ref.abs().max()), float(e.pow(2).mean().sqrt())))
        (a0, m0, r0), (a1, m1, r1) = stats
        accs = -(-Cc // (16 if mode == 4 else 8)) * (R * R if not general else 2 if mode == 4 else 9)
        assert a0 < -0.3e-8 * accs, (mode, stats)                      # raw sums shrink (two main accumulators halve it)
        assert abs(a1) <= max(0.3 * abs(a0), 1e-7) and abs(a1) <= 7e-7 and m1 < m0 and r1 < r0, (mode, stats)
        assert m1 <= FP32_TOL / 2
    xi = torch.randint(0, 10, (2, Cc, H, H), generator=g).float().cuda()
    ones = torch.ones(32, Cc, R, R).cuda()
    want = torch.nn.functional.conv2d(xi.double(), ones.double(), None, 2 if general else 1, 1 if general else (R - 1) // 2)
    assert torch.equal(T.TcConv(ones, mode=4, general=general)(xi, **kw).double(), want)
    assert rel_err(T.TcConv(ones, mode=4, general=general, unbiased=True)(xi, **kw).cpu().numpy(), want.cpu().numpy()) <= FP32_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("B,Cc,K,H,W,R", [(9, 64, 64, 56, 56, 3), (70, 24, 40, 14, 14, 3), (2, 256, 256, 14, 14, 3), (16, 32, 32, 28, 28, 1),
                                           (3, 520, 256, 12, 12, 1), (5, 33, 130, 8, 10, 3)])
def test_fp16_parts_loaders_runs_and_range(T, B, Cc, K, H, W, R, monkeypatch):
    """Mode 4.  (1) Its two input loaders (bulk-tensor boxes filled by a producer thread; the cp.async ring) put
    the same values in the same places: every output bit agrees, whatever the depth of the rings.  (2) Cutting
    the channel blocks into runs that the epilogue adds in fp32 changes the rounding, not the result: within the
    bar, and no farther from fp64 than one run.  (3) The power-of-two scaling into fp16's range makes the result
    independent of the magnitude of input and filter: inputs of 1e-6 and 1e+20 times the same data give the
    same relative error.  (4) The output's recorded largest magnitude is the true one, and a call that is handed
    it skips its own pass over the input without changing a bit."""
    from tdc_b200 import tc
    x, w = draw_core(2500 + B + Cc + H, B, Cc, K, H, W, R)
    xd, wd = x.cuda(), w.cuda()
    ref = torch.nn.functional.conv2d(xd.double(), wd.double(), None, 1, (R - 1) // 2)
    conv = T.TcConv(wd, mode=4)
    y = conv(xd)
    err = rel_err(y.cpu().numpy(), ref.cpu().numpy())
    assert err <= FP32_TOL
    for knobs in ({"TDC_TC_BULK": "0"}, {"TDC_TC_BULK": "1"}, {"TDC_TC_BULK": "1", "TDC_TC_DEPTH": "2"}, {"TDC_TC_BULK": "0", "TDC_TC_MT": "1"},
                  {"TDC_TC_BULK": "1", "TDC_TC_MT": "1", "TDC_TC_NBUF": "1"}, {"TDC_TC_NS": "2"}, {"TDC_TC_TAIL": "0"}, {"TDC_TC_PDL": "0"}, {"TDC_TC_LW": "8"}, {"TDC_TC_LW": "12"},
                  {"TDC_TC_LW": "12", "TDC_TC_BULK": "0"}):
        for k, v in knobs.items():
            monkeypatch.setenv(k, v)
        assert torch.equal(conv(xd), y), knobs
        for k in knobs:
            monkeypatch.delenv(k)
    for chain in ("9", "18", "0"):
        monkeypatch.setenv("TDC_TC_CHAIN", chain)
        e2 = rel_err(conv(xd).cpu().numpy(), ref.cpu().numpy())
        assert e2 <= FP32_TOL and (chain == "0" or e2 <= 1.5 * err + 2e-7), (chain, e2, err)
    monkeypatch.delenv("TDC_TC_CHAIN")
    for sx, sw in ((1e-6, 1.0), (1e20, 1e-9), (3e4, 7e3)):
        ys = T.TcConv(wd * sw, mode=4)(xd * sx)
        assert rel_err(ys.cpu().numpy(), (ref * (sx * sw)).cpu().numpy()) <= max(2 * err, 2e-6), (sx, sw)
    # the scale taken from the true maximum instead of a sample: the same result to rounding
    assert rel_err(T.TcConv(wd, mode=4, exact_range=True)(xd).cpu().numpy(), ref.cpu().numpy()) <= max(2 * err, 2e-6)
    # an outlier 100 times the largest value, which a sample of 4096 elements will not hit: inside the headroom
    xo = xd.clone()
    xo.view(-1)[12345 % xo.numel()] = 100.0 * float(xd.abs().max())
    refo = torch.nn.functional.conv2d(xo.double(), wd.double(), None, 1, (R - 1) // 2)
    assert rel_err(conv(xo).cpu().numpy(), refo.cpu().numpy()) <= FP32_TOL and tc.status() == 0
    assert float(y._tdc_absmax.max()) == float(y.abs().max())
    y_next = T.TcConv(torch.eye(K).view(K, K, 1, 1).cuda().contiguous(), mode=4)
    plain = y.clone()                                     # no recorded magnitude: the call makes its own pass
    assert torch.equal(y_next(y), y_next(plain))
    assert tc.status() == 0
