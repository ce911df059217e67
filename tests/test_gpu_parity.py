"""Parity of the CUDA path with the oracle, through the C ABI, on a B200."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from helpers import FP32_TOL, SWEEP, draw_block, draw_core, load_cases, load_cfg1, rel_err

pytestmark = pytest.mark.gpu
CASES = load_cases()


@pytest.fixture(scope="module")
def T(built):
    import tdc_b200
    assert torch.cuda.is_available(), "these tests need a GPU"
    return tdc_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ---- golden fixtures made by the reference's own TKConv2dC --------------------------------
@pytest.mark.parametrize("name", sorted(CASES))
def test_core_step_against_reference_outputs(T, name):
    c = CASES[name]; m = c["meta"]
    z2 = T.core_conv2d(dev(c["z1"]), dev(c["core"]), m["stride"], m["pad"]).cpu().numpy()
    assert z2.shape == c["z2"].shape
    assert rel_err(z2, c["z2"]) <= FP32_TOL
    crsk = T.permute_weights(dev(c["core"]))
    assert np.array_equal(crsk.cpu().numpy(), c["core"].transpose(1, 2, 3, 0))
    z2b = T.core_conv2d(dev(c["z1"]), crsk, m["stride"], m["pad"], w_layout=T.W_CRSK).cpu().numpy()
    assert rel_err(z2b, c["z2"]) <= FP32_TOL


@pytest.mark.parametrize("name", sorted(CASES))
def test_tucker_block_against_reference_outputs(T, name):
    c = CASES[name]; m = c["meta"]
    y = T.tk_block(dev(c["x"]), dev(c["first"]), dev(c["core"]), dev(c["last"]),
                   None if c["bias"] is None else dev(c["bias"]), m["stride"], m["pad"]).cpu().numpy()
    assert y.shape == c["y"].shape
    assert rel_err(y, c["y"]) <= FP32_TOL


def test_cfg1_single_core_conv(T):
    x, core, z2 = load_cfg1()
    y = T.core_conv2d(dev(x), dev(core), 1, 1).cpu().numpy()
    assert rel_err(y, z2) <= FP32_TOL


# ---- bit-exact twin: same summation order on the CPU ---------------------------------------
TILES = [
    # th tw tc tn nog gy gx imgs ks kc
    (2, 7, 8, 8, 4, 2, 2, 1, 1, 1), (2, 8, 4, 8, 8, 2, 1, 1, 1, 1), (1, 7, 8, 8, 4, 4, 2, 1, 2, 1), (1, 8, 16, 4, 8, 3, 2, 1, 4, 1),
    (2, 7, 4, 4, 8, 7, 2, 2, 1, 1), (2, 8, 8, 4, 16, 7, 2, 1, 2, 1), (1, 7, 8, 4, 4, 14, 2, 2, 2, 1), (1, 8, 8, 8, 8, 14, 2, 1, 1, 1),
    (2, 7, 6, 8, 8, 1, 1, 1, 3, 1), (4, 7, 8, 4, 8, 2, 2, 1, 1, 1), (4, 8, 8, 4, 16, 4, 2, 1, 1, 1), (4, 7, 4, 4, 16, 4, 2, 2, 1, 1),
    (4, 8, 16, 4, 8, 1, 1, 1, 2, 1),
    # chunks split over the CTAs of a cluster (kc), alone and together with slices (ks); 20 channels
    # in chunks of 4 = 5 chunks, so with kc = 4 the ranks get 2, 2, 1 and 0 chunks
    (1, 7, 4, 4, 4, 2, 2, 1, 1, 2), (1, 8, 4, 4, 8, 7, 2, 1, 2, 4), (2, 7, 4, 4, 8, 7, 2, 2, 1, 4), (4, 7, 2, 4, 8, 2, 2, 1, 2, 8),
    (1, 7, 8, 8, 4, 14, 2, 1, 4, 2),
]


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("stride", [1, 2])
def test_bit_exact_against_ordered_oracle(T, tile, stride):
    B, R1, R2, H, W = 3, 20, 36, 14, 14
    x, w = draw_core(100 + sum(tile), B, R1, R2, H, W)
    t = T.Tile(*tile)
    y = T.core_conv2d(x.cuda(), w.cuda(), stride, 1, tile=t).cpu().numpy()
    ref = O.conv2d_f32_sliced(x.numpy(), w.numpy(), tc=t.tc, ks=t.ks, kc=t.kc, pad=1, stride=stride)
    assert np.array_equal(y, ref), (tile, stride, rel_err(y, ref))
    # and run-to-run identical
    y2 = T.core_conv2d(x.cuda(), w.cuda(), stride, 1, tile=t).cpu().numpy()
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("k,stride,pad", [(1, 1, 0), (1, 2, 0), (5, 1, 2), (7, 2, 3), (3, 1, 0), (3, 1, 2), (2, 1, 0)])
def test_other_filters_against_arbiter(T, k, stride, pad):
    x, w = draw_core(200 + k * 10 + stride, 2, 11, 13, 17, 15, k)
    y = T.core_conv2d(x.cuda(), w.cuda(), stride, pad).cpu().numpy()
    ref = O.conv2d_f64(x.numpy(), w.numpy(), pad=pad, stride=stride)
    assert y.shape == ref.shape and rel_err(y, ref) <= FP32_TOL


@pytest.mark.parametrize("B,R1,R2,H,W", [(1, 1, 1, 1, 1), (1, 3, 33, 2, 3), (2, 33, 3, 5, 7), (7, 8, 8, 3, 1), (1, 9, 5, 1, 9),
                                         (5, 4, 4, 7, 7), (2, 16, 16, 15, 57), (1, 32, 32, 56, 56)])
def test_ragged_and_tiny_shapes(T, B, R1, R2, H, W):
    x, w = draw_core(300 + B + R1 + H, B, R1, R2, H, W)
    y = T.core_conv2d(x.cuda(), w.cuda(), 1, 1).cpu().numpy()
    ref = O.conv2d_f64(x.numpy(), w.numpy(), pad=1)
    assert rel_err(y, ref) <= FP32_TOL


def test_bias_and_relu_epilogue(T):
    x, w = draw_core(42, 2, 8, 12, 9, 9)
    b = torch.randn(12, generator=torch.Generator().manual_seed(1))
    y = T.conv2d(x.cuda(), w.cuda(), b.cuda(), 1, 1, relu=True).cpu().numpy()
    ref = O.conv2d_f64(x.numpy(), w.numpy(), b.numpy(), pad=1, relu=True)
    assert rel_err(y, ref) <= FP32_TOL and (y >= 0).all() and (y == 0).any()


# ---- the reference drivers' own check: integer inputs, all-ones weights => exact ------------
@pytest.mark.parametrize("C_,N,H", [(32, 32, 56), (64, 64, 56), (96, 64, 28), (192, 160, 7), (128, 96, 14)])
def test_integer_inputs_are_exact(T, C_, N, H):
    rng = np.random.default_rng(C_ + H)
    inp = rng.integers(0, 10, (1, C_, H, H)).astype(np.float32)
    k = np.ones((C_, 3, 3, N), np.float32)            # the reference kernel's [c][r][s][n]
    y = T.core_conv2d(dev(inp), dev(k), 1, 1, w_layout=T.W_CRSK).cpu().numpy()
    ref = O.conv2d_f64(inp, k, pad=1, w_layout=O.W_CRSK)
    assert np.array_equal(y, ref)
    if H <= 14:
        th, tw, tc = {7: (2, 2, 16), 14: (1, 2, 32)}[H]  # the shipped tiles of those two shapes
        assert np.array_equal(y[0], O.ref_tiled(inp[0], k, th, tw, tc))


# ---- full benchmark sizes: every sweep shape against the oracle / by properties --------------
@pytest.mark.parametrize("H,R1,R2", SWEEP)
def test_sweep_batch1_against_arbiter(T, H, R1, R2):
    i = SWEEP.index((H, R1, R2))
    x, w = draw_core(2000 + i, 1, R1, R2, H, H)
    y = T.core_conv2d(x.cuda(), w.cuda(), 1, 1).cpu().numpy()
    assert rel_err(y, O.conv2d_f64(x.numpy(), w.numpy(), pad=1)) <= FP32_TOL


@pytest.mark.parametrize("H,R1,R2", SWEEP)
def test_sweep_batch64_properties(T, H, R1, R2):
    """At B=64 the oracle is too slow to run whole; check (1) four sampled images against the
    arbiter, (2) batch independence: image b of the batched call equals the same image run alone
    with the same tile (bit-exact), (3) linearity in x within tolerance."""
    i = SWEEP.index((H, R1, R2))
    x, w = draw_core(2100 + i, 64, R1, R2, H, H)
    xd, wd = x.cuda(), T.permute_weights(w.cuda())
    t = T.select_tile(64, R1, H, H, R2, 3, 3, 1, 1)
    y = T.core_conv2d(xd, wd, 1, 1, w_layout=T.W_CRSK, tile=t)
    sel = [0, 21, 42, 63]
    ref = O.conv2d_f64(x[sel].numpy(), w.numpy(), pad=1)
    assert rel_err(y[sel].cpu().numpy(), ref) <= FP32_TOL
    if t.imgs == 1:
        one = T.core_conv2d(xd[5:6].contiguous(), wd, 1, 1, w_layout=T.W_CRSK, tile=t)
        assert torch.equal(one[0], y[5])
    y2 = T.core_conv2d((2.0 * xd).contiguous(), wd, 1, 1, w_layout=T.W_CRSK, tile=t)
    assert torch.equal(y2, 2.0 * y)     # scaling by a power of two is exact in fp32
    ys = T.core_conv2d((xd + xd.flip(0)).contiguous(), wd, 1, 1, w_layout=T.W_CRSK, tile=t)
    lin = (y + y.flip(0))
    assert float((ys - lin).abs().max() / lin.abs().max()) <= FP32_TOL


def test_stride2_sweep_shapes(T):
    for (H, R1, R2) in [(56, 64, 64), (28, 96, 96), (14, 160, 160)]:
        x, w = draw_core(2200 + H, 2, R1, R2, H, H)
        y = T.core_conv2d(x.cuda(), w.cuda(), 2, 1).cpu().numpy()
        assert rel_err(y, O.conv2d_f64(x.numpy(), w.numpy(), pad=1, stride=2)) <= FP32_TOL


# ---- module and layer objects ---------------------------------------------------------------
def test_module_matches_reference_forward(T):
    class HP:
        ranks = {"l": [24, 16]}
    torch.manual_seed(3)
    m = T.TKConv2dC_B200(32, 48, 3, stride=1, padding=1, bias=True, hp_dict=HP, name="l")
    with torch.no_grad():
        m.bias.normal_()
    ref = O.TKConv2dCRef(m.first_kernel.detach().clone(), m.core_kernel.detach().clone(), m.last_kernel.detach().clone(),
                         m.bias.detach().clone(), 1, 1)
    x = torch.randn(4, 32, 28, 28)
    m = m.cuda()
    with torch.no_grad():
        y = m(x.cuda())
        y_ref, feats_ref = ref.forward_features(x)
        y2, feats = m.forward_features(x.cuda())
    assert rel_err(y.cpu().numpy(), y_ref.numpy()) <= FP32_TOL
    assert rel_err(y2.cpu().numpy(), y_ref.numpy()) <= FP32_TOL
    for a, b in zip(feats, feats_ref):
        assert rel_err(a.cpu().numpy(), b.numpy()) <= FP32_TOL
    # weights changed in place are picked up (the channel-last copy is refreshed)
    with torch.no_grad():
        m.core_kernel.mul_(2.0)
        assert rel_err(m(x.cuda()).cpu().numpy(), (2 * (y_ref - ref.bias.view(1, -1, 1, 1)) + ref.bias.view(1, -1, 1, 1)).numpy()) <= FP32_TOL


def test_layer_objects_with_host_buffers(T):
    """tdc_conv / tdc_tkconv mirror Conv::initialize/forward and TkConv of the reference's
    end-to-end skeleton; forward_host is the drivers' copy-in / run / copy-out."""
    lib = T.lib
    x, first, core, last, b = draw_block(77, 2, 16, 24, 8, 12, 14, 14, 3, bias=True)
    xn = x.numpy()
    fp = lambda a: a.ctypes.data_as(C.c_void_p)
    h = C.c_void_p()
    wn = core.numpy()
    z1 = O.conv2d_f64(xn, first.numpy())
    assert lib.tdc_conv_create(C.byref(h), 2, 8, 14, 14, 12, 1, 3, 3, 1, fp(wn), None) == 0
    out = np.empty((2, 12, 14, 14), np.float32)
    assert lib.tdc_conv_forward_host(h, fp(z1), fp(out)) == 0
    assert rel_err(out, O.conv2d_f64(z1, wn, pad=1)) <= FP32_TOL
    # the variant that leaves the synchronise to the caller, on a stream of the caller's: pinned buffers, same bits
    side = torch.cuda.Stream()
    zin, zout = torch.from_numpy(z1).pin_memory(), torch.empty(2, 12, 14, 14).pin_memory()
    assert lib.tdc_conv_forward_host_async(h, C.c_void_p(zin.data_ptr()), C.c_void_p(zout.data_ptr()), C.c_void_p(side.cuda_stream)) == 0
    side.synchronize()
    assert np.array_equal(zout.numpy(), out)
    lib.tdc_conv_destroy(h)
    # all-ones weights when none are given, as the reference fills them (Conv.cu:88-91)
    assert lib.tdc_conv_create(C.byref(h), 1, 4, 6, 6, 5, 1, 3, 3, 1, None, None) == 0
    xi = np.random.default_rng(0).integers(0, 10, (1, 4, 6, 6)).astype(np.float32)
    out = np.empty((1, 5, 6, 6), np.float32)
    assert lib.tdc_conv_forward_host(h, fp(xi), fp(out)) == 0
    assert np.array_equal(out, O.conv2d_f64(xi, np.ones((5, 4, 3, 3), np.float32), pad=1))
    lib.tdc_conv_destroy(h)

    tk = C.c_void_p()
    f2, l2, bn = first.numpy().reshape(8, 16), last.numpy().reshape(24, 12), b.numpy()
    assert lib.tdc_tkconv_create(C.byref(tk), 2, 16, 8, 12, 24, 14, 14, 3, 3, 1, 2, fp(f2), fp(wn), fp(l2), fp(bn)) == 0
    out = np.empty((2, 24, 7, 7), np.float32)
    assert lib.tdc_tkconv_forward_host(tk, fp(xn), fp(out)) == 0
    ref, _, _ = O.tk_block(xn, f2, wn, l2, bn, pad=1, stride=2, f64=True)
    assert rel_err(out, ref) <= FP32_TOL
    # the same layer as ONE tensor-core launch on the merged filter (here a strided 3x3: the gathering plan), and back
    for mode in (4, 3):
        assert lib.tdc_tkconv_set_precision(tk, mode) == 0
        out2 = np.empty_like(out)
        assert lib.tdc_tkconv_forward_host(tk, fp(xn), fp(out2)) == 0
        assert rel_err(out2, ref) <= FP32_TOL and not np.array_equal(out2, out)
    assert lib.tdc_tkconv_set_precision(tk, 0) == 0
    out3 = np.empty_like(out)
    assert lib.tdc_tkconv_forward_host(tk, fp(xn), fp(out3)) == 0 and np.array_equal(out3, out)
    lib.tdc_tkconv_destroy(tk)


def test_errors_on_device(T):
    from tdc_b200 import _lib
    x = torch.zeros(1, 8, 5, 5).cuda(); w = torch.zeros(4, 8, 3, 3).cuda()
    with pytest.raises(T.TdcError) as e:
        T.core_conv2d(x, w, 3, 1)
    assert e.value.code == _lib.ERR_UNSUPPORTED
    with pytest.raises(T.TdcError) as e:
        T.core_conv2d(x, w, 1, 1, tile=T.Tile(2, 7, 8, 8, 4, 64, 8, 1, 1, 1))
    assert e.value.code == _lib.ERR_TILE
    with pytest.raises(T.TdcError) as e:
        T.tk_block(x, torch.zeros(4, 8).cuda(), torch.zeros(4, 4, 3, 3).cuda(), torch.zeros(6, 4).cuda(),
                   workspace=torch.empty(16, dtype=torch.uint8).cuda())
    assert e.value.code == _lib.ERR_WORKSPACE
    with pytest.raises(T.TdcError):
        T.core_conv2d(x.double(), w, 1, 1)
    info = T.tile_info((64, 64, 56, 56, 64, 3, 3, 1, 1), T.Tile())
    assert info.threads > 0 and info.ctas_per_sm >= 1 and info.regs_per_thread > 0
