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
    for H, R in ((56, 32), (28, 64), (28, 128), (14, 256), (7, 512)):
        assert not tc.worthwhile(1, R, H, H, R, 3)
    # batch 64: tensor cores for every sweep shape
    for H, R in ((56, 32), (28, 64), (14, 128), (7, 256), (7, 512)):
        assert tc.worthwhile(64, R, H, H, R, 3)
    # the Tucker blocks at batch 32: every step but the 1x1 steps of the 7x7 block (1568 positions)
    assert tc.worthwhile(32, 64, 56, 56, 32, 1) and tc.worthwhile(32, 128, 14, 14, 128, 3) and tc.worthwhile(32, 256, 7, 7, 256, 3)
    assert not tc.worthwhile(32, 512, 7, 7, 256, 1) and not tc.worthwhile(32, 256, 7, 7, 512, 1)
    # many positions but hardly any arithmetic
    assert not tc.worthwhile(64, 3, 56, 56, 8, 1)
