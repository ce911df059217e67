"""Which kernel family a convolution goes to (tdc_b200/tc.py, tdc_b200/dispatch.py): the host-side rules, no GPU."""
import pytest


@pytest.fixture(scope="module")
def tc(built):
    from tdc_b200 import tc
    return tc


def test_one_pass_plan_covers_same_convs_and_strided_1x1(tc):
    assert tc.supported(3, 3, 1, 1, 56) and tc.supported(1, 1, 1, 0, 7)
    assert tc.supported(1, 1, 2, 0, 56)                      # the shortcut convolution
    assert not tc.supported(3, 3, 2, 1, 56)                  # a strided core needs the gathering plan
    assert not tc.supported(3, 3, 1, 0, 56) and not tc.supported(5, 5, 1, 2, 56) and not tc.supported(3, 1, 1, 1, 56)
    assert not tc.supported(3, 3, 1, 1, 300)                 # image width limit of the position tiles
    assert tc.general_supported(7, 7, 2, 3, 112) and tc.general_supported(3, 3, 2, 1, 28)
    assert not tc.general_supported(17, 17, 1, 8, 10) and not tc.general_supported(3, 3, 1, 16, 10)


def test_tensor_cores_only_where_they_fill_the_gpu(tc):
    # batch-1 layers: the fp32 kernel with clusters (too few positions or too little arithmetic for 128-position tiles)
    for H, R in ((56, 32), (28, 64), (14, 128), (14, 256), (7, 512)):
        assert not tc.worthwhile(1, R, H, H, R, 3)
    assert tc.worthwhile(1, 64, 56, 56, 64, 3)                       # 26 position tiles, 0.23 GFLOP: measured 16 vs 19 us
    # a few images are enough for the 3x3 layers with at least three position tiles
    assert tc.worthwhile(2, 32, 56, 56, 32, 3) and tc.worthwhile(4, 128, 14, 14, 128, 3) and tc.worthwhile(8, 512, 7, 7, 512, 3)
    assert tc.worthwhile(2, 256, 14, 14, 256, 3)                                                  # measured 27 vs 45 us
    assert not tc.worthwhile(2, 256, 7, 7, 256, 3) and not tc.worthwhile(4, 512, 7, 7, 512, 3)    # 33 vs 23 us, a tie
    # batch 64: tensor cores for every sweep shape
    for H, R in ((56, 32), (28, 64), (14, 128), (7, 256), (7, 512)):
        assert tc.worthwhile(64, R, H, H, R, 3)
    # the Tucker blocks at batch 32: every step (the first 1x1 step of the 7x7 block, 12 tiles and 512 channels to walk, is a tie)
    assert tc.worthwhile(32, 64, 56, 56, 32, 1) and tc.worthwhile(32, 128, 14, 14, 128, 3) and tc.worthwhile(32, 256, 7, 7, 256, 3)
    assert tc.worthwhile(32, 256, 7, 7, 512, 1)                                                   # measured 46 vs 32 us
    # 1x1 layers with few tiles (tensor cores vs fp32, us): four tiles with some arithmetic, wide outputs from three
    # tiles on, and up to 512 channels to walk whatever the tile count when the arithmetic is there
    assert tc.worthwhile(8, 512, 7, 7, 2048, 1) and not tc.worthwhile(8, 2048, 7, 7, 512, 1)      # 131 vs 88
    assert tc.worthwhile(16, 256, 14, 14, 128, 1) and tc.worthwhile(8, 256, 14, 14, 128, 1)       # 22 vs 44, 22 vs 25
    assert tc.worthwhile(16, 2048, 7, 7, 512, 1) and tc.worthwhile(4, 1024, 14, 14, 256, 1)       # 133 vs 147, 51 vs 88
    assert not tc.worthwhile(2, 1024, 14, 14, 256, 1) and not tc.worthwhile(1, 1024, 7, 7, 512, 1)  # 51 vs 43, 70 vs 61
    assert tc.worthwhile(32, 1024, 7, 7, 512, 1)                                                  # 74 vs 123
    # many positions but hardly any arithmetic
    assert not tc.worthwhile(64, 3, 56, 56, 8, 1)


def test_thresholds_against_the_recorded_timings(tc):
    """tests/golden/tc_vs_fp32_times_b200.json: 420 layers timed on both kernels on a B200 (make_tc_vs_fp32_times.py
    beside it).  Summed over the file, the time of the kernel the rule picks stays within 2 % of the time of the faster
    kernel per layer, for the 3x3 and for the 1x1 layers, and no single pick costs more than 1.7x."""
    import json
    import os
    from helpers import ROOT
    rows = json.load(open(os.path.join(ROOT, "tests", "golden", "tc_vs_fp32_times_b200.json")))
    assert len(rows) == 420
    for R, bar in ((3, 1.01), (1, 1.02)):
        picked = best = 0.0
        for (r, C, K, H, B, t_tc, t_fp) in rows:
            if r != R:
                continue
            mine = t_tc if tc.worthwhile(B, C, H, H, K, r) else t_fp
            assert mine <= 1.7 * min(t_tc, t_fp), (r, C, K, H, B, t_tc, t_fp)
            picked += mine
            best += min(t_tc, t_fp)
        assert picked <= bar * best, (R, picked / best)


def test_block_size_by_position_count(built):
    """tdc_tc_pick_nt: the default block (128 / 64 / 32 output channels by K) for layers with many position tiles,
    smaller blocks where the positions alone leave SMs idle — a host-side rule, no GPU."""
    import ctypes as C
    import tdc_b200 as T
    from tdc_b200 import _lib
    pick = lambda K, pos, mode=3: T.lib.tdc_tc_pick_nt(K, mode, pos, 148)
    assert pick(64, 64 * 57 * 57) == 64 and pick(128, 64 * 29 * 29) == 128 and pick(32, 64 * 57 * 57) == 32
    assert pick(128, 32 * 29 * 29) == 128        # 211 tiles fill 148 SMs: the default stays
    assert pick(512, 64 * 8 * 8) == 128          # 7x7x512 at batch 64: 128 tiles of 128-channel blocks already
    assert pick(256, 64 * 8 * 8) == 64           # 7x7x256 at batch 64: 64 tiles -> 128 tiles of 64-channel blocks
    assert pick(256, 32 * 8 * 8) == 32           # the core of the 7x7 Tucker block at batch 32
    p = _lib.TcPlan()
    assert T.lib.tdc_tc_plan_make_nt(256, 256, 3, 3, 3, 0, 64, C.byref(p)) == 0
    assert (p.nt, p.n_ocb, p.nkb) == (64, 4, 32) and p.weights_bytes == 4 * 2 * 9 * 8 * 64 * 32 * 4
    assert T.lib.tdc_tc_plan_make_nt(256, 256, 3, 3, 3, 0, 48, C.byref(p)) == _lib.ERR_UNSUPPORTED
    assert T.lib.tdc_tc_plan_make_nt(3, 64, 7, 7, 3, 1, 32, C.byref(p)) == 0 and (p.general, p.nt, p.n_ocb) == (1, 32, 2)
