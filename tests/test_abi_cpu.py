"""Host-side checks of the C ABI that need no GPU: the library loads, exports every symbol
include/tdc_b200.h declares, rejects bad arguments with status codes, and the selector runs
from a hand-filled device description."""
import ctypes as C
import os
import re

import pytest

from helpers import SWEEP

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def T(built):
    import tdc_b200
    return tdc_b200


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tdc_b200.h")).read()
    return sorted(set(re.findall(r"TDC_API[^;(]*?\b(tdc_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(T):
    names = declared_symbols()
    assert len(names) >= 20
    raw = C.CDLL(T.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), n
    from tdc_b200 import _lib
    assert sorted(_lib.EXPORTS) == names


def test_version_and_error_string(T):
    assert T.lib.tdc_version() >= 100
    assert isinstance(T.lib.tdc_last_error_string(), bytes)


def test_bad_arguments_are_status_codes_not_crashes(T):
    from tdc_b200 import _lib
    lib = T.lib
    # NULL pointers are caught before any CUDA call
    assert lib.tdc_core_conv2d_f32(None, None, None, 1, 1, 1, 1, 1, 1, 1, 0, 1, 0, None, None) == _lib.ERR_NULL
    assert lib.tdc_permute_weights(None, None, 1, 1, 1, 1, None) == _lib.ERR_NULL
    assert lib.tdc_select_tile(1, 1, 1, 1, 1, 1, 1, 0, 1, None, None) == _lib.ERR_NULL
    t = T.Tile()
    dev = T.B200
    sel = lambda *a: lib.tdc_select_tile(*a, C.byref(dev), C.byref(t))
    assert sel(0, 32, 56, 56, 32, 3, 3, 1, 1) == _lib.ERR_SHAPE          # empty batch
    assert sel(1, 32, 2, 2, 32, 5, 5, 0, 1) == _lib.ERR_SHAPE            # filter larger than input
    assert sel(1, 32, 56, 56, 32, 3, 3, 1, 3) == _lib.ERR_UNSUPPORTED    # stride 3
    assert sel(1, 32, 56, 56, 32, 9, 9, 4, 1) == _lib.ERR_UNSUPPORTED    # 9x9
    assert b"stride" in lib.tdc_last_error_string() or b"filter" in lib.tdc_last_error_string()
    assert lib.tdc_tk_block_workspace_bytes(0, 1, 1, 1, 1, 1, 1, 3, 3, 1, 1) == 0
    assert lib.tdc_tk_block_workspace_bytes(2, 8, 5, 5, 4, 6, 8, 3, 3, 1, 1) >= 4 * (2 * 4 * 25 + 2 * 6 * 25)


def test_every_refusal_leaves_its_reason_in_the_one_error_string(T):
    """All entry points share one thread-local message (tdc_last_error_string; tdc_tc_last_error_string is the same
    text): each non-zero status below must leave a message of its own there, not the previous call's."""
    from tdc_b200 import _lib
    lib = T.lib
    one = C.c_void_p(16)         # a non-NULL, 16-byte aligned stand-in that no check dereferences before refusing
    odd = C.c_void_p(20)         # ... and one that is not 16-byte aligned
    h = C.c_void_p()
    plan = _lib.TcPlan()
    assert lib.tdc_tc_plan_make(8, 8, 3, 3, 4, C.byref(plan)) == 0
    cases = [
        ("pool NULL", lambda: lib.tdc_pool2d_f32(None, None, 1, 1, 4, 4, 2, 2, 0, 2, 0, None), _lib.ERR_NULL, b"tdc_pool2d_f32"),
        ("pool window", lambda: lib.tdc_pool2d_f32(one, one, 1, 1, 4, 4, 2, 2, 2, 2, 0, None), _lib.ERR_SHAPE, b"padding"),
        ("pool mode", lambda: lib.tdc_pool2d_f32(one, one, 1, 1, 4, 4, 2, 2, 0, 2, 7, None), _lib.ERR_UNSUPPORTED, b"mode 7"),
        ("affine NULL", lambda: lib.tdc_affine_relu_f32(None, None, None, None, 1, 1, 1, 1, 1, 0, None), _lib.ERR_NULL, b"tdc_affine_relu_f32"),
        ("affine stride", lambda: lib.tdc_affine_relu_f32(one, one, None, None, 2, 4, 9, 8, 36, 0, None), _lib.ERR_SHAPE, b"strides"),
        ("conv create", lambda: lib.tdc_conv_create(C.byref(h), 0, 1, 1, 1, 1, 0, 1, 1, 1, None, None), _lib.ERR_SHAPE, b"tdc_conv_create"),
        ("conv precision", lambda: lib.tdc_conv_set_precision(None, 3), _lib.ERR_NULL, b"tdc_conv_set_precision"),
        ("conv forward", lambda: lib.tdc_conv_forward(None, None, None, None), _lib.ERR_NULL, b"tdc_conv_forward"),
        ("host forward", lambda: lib.tdc_conv_forward_host_async(None, None, None, None), _lib.ERR_NULL, b"tdc_conv_forward_host_async"),
        ("tkconv create", lambda: lib.tdc_tkconv_create(C.byref(h), 1, 1, 1, 1, 1, 1, 1, 3, 3, 0, 1, None, None, None, None), _lib.ERR_SHAPE, b"tdc_tkconv_create"),
        ("tkconv forward", lambda: lib.tdc_tkconv_forward(None, None, None, None), _lib.ERR_NULL, b"tdc_tkconv_forward"),
        ("tc plan", lambda: lib.tdc_tc_plan_make(8, 8, 5, 5, 3, C.byref(plan)), _lib.ERR_UNSUPPORTED, b"5x5"),
        ("tc unaligned filter", lambda: lib.tdc_conv2d_tc(C.byref(plan), one, odd, one, 1, 4, 4, None, 0, None), _lib.ERR_UNSUPPORTED, b"16-byte"),
        ("tc prepare unaligned", lambda: lib.tdc_tc_prepare_weights(C.byref(plan), one, 0, odd, None), _lib.ERR_UNSUPPORTED, b"16-byte"),
        ("tc flags", lambda: lib.tdc_conv2d_tc(C.byref(plan), one, one, one, 1, 4, 4, None, 0x800, None), _lib.ERR_UNSUPPORTED, b"flag"),
        ("tc ranged other mode", None, None, None),
    ]
    for name, call, want, needle in cases:
        if call is None:
            continue
        got = call()
        msg = lib.tdc_last_error_string()
        assert got == want and needle in msg, (name, got, msg)
        assert lib.tdc_tc_last_error_string() == msg, name
    p3 = _lib.TcPlan()
    assert lib.tdc_tc_plan_make(8, 8, 3, 3, 3, C.byref(p3)) == 0
    assert lib.tdc_conv2d_tc_ranged(C.byref(p3), one, one, one, 1, 4, 4, None, 0, None, one, None) == _lib.ERR_UNSUPPORTED
    assert b"y_absmax" in lib.tdc_last_error_string()


def test_tensor_core_plans_are_host_arithmetic(T):
    """The plan makers run on the host alone: block sizes, channel blocks and prepared-filter sizes of the one-pass,
    gathering and strided-row plans; the strided-row plan's column phase (1 with an odd padding at stride 2 when the shift
    keeps 2 or 4 taps); what each refusal says."""
    from tdc_b200 import _lib
    from tdc_b200 import tc
    lib = T.lib
    p = _lib.TcPlan()
    assert lib.tdc_tc_plan_make(64, 64, 3, 3, 4, C.byref(p)) == 0
    assert (p.nt, p.cb, p.nkb, p.n_ocb, p.hl, p.general) == (64, 16, 4, 1, 2, 0)
    assert lib.tdc_tc_plan_make_general(3, 64, 7, 7, 3, C.byref(p)) == 0 and (p.general, p.nkb) == (1, 19)
    for (Cc, K, R, S, stride, pad, phase, nkb, taps) in ((3, 64, 7, 7, 2, 3, 1, 3, 4), (64, 128, 3, 3, 2, 1, 1, 24, 2), (64, 128, 3, 3, 2, 0, 0, 24, 2),
                                                        (8, 8, 4, 4, 2, 1, 0, 4, 2), (8, 8, 3, 7, 4, 1, 0, 6, 2), (16, 32, 8, 8, 2, 3, 0, 16, 4)):
        assert tc.strided_rows(S, stride)
        assert lib.tdc_tc_plan_make_strided(Cc, K, R, S, stride, pad, 4, 0, C.byref(p)) == 0, lib.tdc_last_error_string()
        assert (p.general, p.stride, p.phase, p.nkb) == (2, stride, phase, nkb), (Cc, K, R, S, stride, pad)
        assert p.weights_bytes == 4 * 2 * taps * 8 * p.nt * p.nkb * p.n_ocb + 4 * (1024 + 64)
    assert not tc.strided_rows(5, 2) and not tc.strided_rows(3, 1)
    for args, needle in (((8, 8, 5, 5, 2, 2, 4, 0), b"2 or 4 column taps"), ((8, 8, 3, 3, 2, 1, 3, 0), b"mode 4"),
                         ((8, 8, 3, 3, 1, 1, 4, 0), b"strides 2..15"), ((8, 8, 3, 3, 2, 1, 4, 48), b"nt 48")):
        assert lib.tdc_tc_plan_make_strided(*args, C.byref(p)) == _lib.ERR_UNSUPPORTED
        assert needle in lib.tdc_last_error_string(), (args, lib.tdc_last_error_string())


@pytest.mark.parametrize("B", [1, 64])
@pytest.mark.parametrize("H,R1,R2", SWEEP)
def test_selector_gives_a_launchable_tile(T, B, H, R1, R2):
    shape = (B, R1, H, H, R2, 3, 3, 1, 1)
    t = T.select_tile(*shape, dev=T.B200)
    assert all(v > 0 for v in t.as_tuple())
    assert t.tc % t.ks == 0
    assert 1 <= t.kc <= 8
    threads = t.ks * t.nog * t.imgs * t.gy * t.gx
    assert 1 <= threads <= (256 if t.tn * t.th * t.tw > 64 else 512)
    if t.imgs > 1:
        assert t.gy * t.th >= H and t.gx * t.tw >= H
    cost, vols = T.tile_cost(shape, t, T.B200)
    assert cost > 0 and vols[2] == B * R2 * H * H and vols[0] > 0 and vols[1] > 0 and vols[3] > 0
    # the selected tile is the argmin among a handful of hand-made alternatives
    for alt in [T.Tile(1, 7, 8, 8, 4, 1, 1, 1, 1, 1), T.Tile(2, 7, 8, 8, 4, 2, 2, 1, 1, 1), T.Tile(1, 8, 4, 4, 8, 1, 1, 1, 1, 1), T.Tile(4, 8, 8, 4, 8, 1, 1, 1, 1, 1)]:
        try:
            c2, _ = T.tile_cost(shape, alt, T.B200)
        except T.TdcError:
            continue
        assert cost <= c2


def test_selector_handles_other_filters(T):
    for shape in [(8, 64, 56, 56, 32, 1, 1, 0, 1), (8, 64, 56, 56, 64, 3, 3, 1, 2), (4, 3, 224, 224, 64, 7, 7, 3, 2),
                  (2, 16, 9, 9, 8, 5, 5, 2, 1), (1, 3, 1, 1, 2, 1, 1, 0, 1)]:
        t = T.select_tile(*shape, dev=T.B200)
        assert all(v > 0 for v in t.as_tuple()), shape


def test_tile_cost_rejects_inconsistent_tiles(T):
    from tdc_b200 import _lib
    shape = (1, 32, 56, 56, 32, 3, 3, 1, 1)
    with pytest.raises(T.TdcError) as e:
        T.tile_cost(shape, T.Tile(2, 7, 8, 8, 4, 2, 2, 3, 1, 1), T.B200)       # imgs>1 without covering the map
    assert e.value.code == _lib.ERR_TILE
    with pytest.raises(T.TdcError) as e:
        T.tile_cost(shape, T.Tile(2, 7, 6, 8, 4, 2, 2, 1, 4, 1), T.B200)       # tc % ks
    assert e.value.code == _lib.ERR_TILE
    with pytest.raises(T.TdcError) as e:
        T.tile_cost(shape, T.Tile(3, 7, 8, 8, 4, 2, 2, 1, 1, 1), T.B200)       # th=3 is not compiled
    assert e.value.code == _lib.ERR_UNSUPPORTED
    with pytest.raises(T.TdcError) as e:
        T.tile_cost(shape, T.Tile(2, 7, 32, 8, 8, 28, 8, 1, 1, 1), T.B200)     # too many threads
    assert e.value.code == _lib.ERR_TILE


def test_module_surface_matches_reference_without_gpu(T):
    """Constructor contract of inference/TKConv.py:23-88: names, shapes, rank order, errors."""
    import torch

    class HP:
        ranks = {"l": [12, 8]}

    m = T.TKConv2dC_B200(16, 24, 3, stride=2, padding=1, bias=True, hp_dict=HP, name="l")
    sd = m.state_dict()
    assert list(sd) == ["first_kernel", "core_kernel", "last_kernel", "bias"]
    assert tuple(sd["first_kernel"].shape) == (8, 16, 1, 1)
    assert tuple(sd["core_kernel"].shape) == (12, 8, 3, 3)
    assert tuple(sd["last_kernel"].shape) == (24, 12, 1, 1)
    assert m.in_rank == 8 and m.out_rank == 12 and m.stride == (2, 2) and m.padding == (1, 1)
    assert "core_conv(in=8, out=12, kernel_size=(3, 3), stride=(2, 2), padding=(1, 1)" in m.extra_repr()
    with pytest.raises(ValueError):
        T.TKConv2dC_B200(16, 24, 3, groups=2, hp_dict=HP, name="l")
    with pytest.raises(ValueError):
        T.TKConv2dC_B200(16, 24, 3, padding_mode="reflect", hp_dict=HP, name="l")
    m2 = T.TKConv2dC_B200(16, 24, 3, bias=False, hp_dict=HP, name="l")
    assert m2.bias is None and "bias" not in m2.state_dict()
    with pytest.raises(T.TdcError):          # no silent CPU path
        m(torch.zeros(1, 16, 8, 8))
