"""The oracle against the reference's own outputs (tests/golden, made by running the
reference's TKConv2dC on CPU) and against the reference drivers' exactness property."""
import numpy as np
import pytest

import oracle as O
from helpers import FP32_TOL, load_cases, load_cfg1, rel_err

CASES = load_cases()


@pytest.mark.parametrize("name", sorted(CASES))
def test_c_oracle_matches_reference_module(built, name):
    c = CASES[name]; m = c["meta"]
    for f64 in (False, True):
        y, z1, z2 = O.tk_block(c["x"], c["first"], c["core"], c["last"], c["bias"], pad=m["pad"], stride=m["stride"], f64=f64)
        assert y.shape == c["y"].shape and z1.shape == c["z1"].shape and z2.shape == c["z2"].shape
        assert rel_err(z1, c["z1"]) <= FP32_TOL
        assert rel_err(z2, c["z2"]) <= FP32_TOL
        assert rel_err(y, c["y"]) <= FP32_TOL


@pytest.mark.parametrize("name", sorted(CASES))
def test_core_step_alone(built, name):
    """The hot step fed with the reference's own intermediate z1."""
    c = CASES[name]; m = c["meta"]
    for fn in (O.conv2d_f32, O.conv2d_f64):
        z2 = fn(c["z1"], c["core"], pad=m["pad"], stride=m["stride"])
        assert rel_err(z2, c["z2"]) <= FP32_TOL
    crsk = np.ascontiguousarray(c["core"].transpose(1, 2, 3, 0))
    assert np.array_equal(O.conv2d_f32(c["z1"], crsk, pad=m["pad"], stride=m["stride"], w_layout=O.W_CRSK),
                          O.conv2d_f32(c["z1"], c["core"], pad=m["pad"], stride=m["stride"]))


@pytest.mark.parametrize("name", sorted(CASES))
def test_torch_restatement_is_the_reference_forward(built, name):
    import torch
    c = CASES[name]; m = c["meta"]
    torch.set_num_threads(1)
    ref = O.TKConv2dCRef(torch.from_numpy(c["first"]), torch.from_numpy(c["core"]), torch.from_numpy(c["last"]),
                         None if c["bias"] is None else torch.from_numpy(c["bias"]), m["stride"], m["pad"])
    y, (z1, z2, _) = ref.forward_features(torch.from_numpy(c["x"]))
    # same torch calls on the same machine type: allow only thread-count reassociation noise
    assert rel_err(y.numpy(), c["y"]) <= 1e-6 and rel_err(z2.numpy(), c["z2"]) <= 1e-6
    assert rel_err(ref.core(z1).numpy(), c["z2"]) <= 1e-6


def test_cfg1_single_core_conv(built):
    x, core, z2 = load_cfg1()
    assert rel_err(O.conv2d_f32(x, core, pad=1), z2) <= FP32_TOL
    assert rel_err(O.conv2d_f64(x, core, pad=1), z2) <= FP32_TOL


def test_sliced_order_is_a_reordering_only(built):
    c = CASES["k3_s1_p1_bias"]
    a = O.conv2d_f32(c["z1"], c["core"], pad=1)
    assert np.array_equal(O.conv2d_f32_sliced(c["z1"], c["core"], tc=4, ks=1, pad=1), a)
    b = O.conv2d_f32_sliced(c["z1"], c["core"], tc=4, ks=2, pad=1)
    assert rel_err(b, a) <= 1e-6 and not np.array_equal(a, b)
    c2 = O.conv2d_f32_sliced(c["z1"], c["core"], tc=2, ks=1, kc=2, pad=1)     # 8 channels: ranks get 2 chunks each
    assert rel_err(c2, a) <= 1e-6 and not np.array_equal(a, c2)
    assert np.array_equal(O.conv2d_f32_sliced(c["z1"], c["core"], tc=4, ks=1, kc=1, pad=1), a)


# Shapes and tiles of the reference's shipped drivers (C, N, H, W, TH, TW, TC): the #defines of
# A100-evaluation/TDC-LAYERS-ORACLE/{32_32_14_14,64_32_7_7,96_64_7_7,32_32_28_28}.cu and one
# ragged tile that exercises the min(TH, H-h0) / min(TW, W-w0) write-back.
@pytest.mark.parametrize("C,N,H,W,TH,TW,TC", [(32, 32, 14, 14, 1, 1, 8), (64, 32, 7, 7, 2, 1, 4), (96, 64, 7, 7, 4, 1, 8),
                                              (32, 32, 28, 28, 1, 2, 8), (16, 8, 13, 11, 3, 4, 8)])
def test_reference_kernel_walk_is_exact_on_integer_inputs(built, C, N, H, W, TH, TW, TC):
    """rand()%10 inputs and all-ones weights (template_benchmark_cudnn.template:418-428) make every
    partial sum a small integer, so any summation order gives the same bits: diff must be 0 (:509)."""
    rng = np.random.default_rng(C * 1000 + H)
    inp = rng.integers(0, 10, (C, H, W)).astype(np.float32)
    k = np.ones((C, 3, 3, N), np.float32)
    tiled = O.ref_tiled(inp, k, TH, TW, TC)
    direct = O.conv2d_f32(inp[None], k, pad=1, w_layout=O.W_CRSK)[0]
    assert np.array_equal(tiled, direct)
    # hand-checkable corner: output(0,0) = sum over channels of the 2x2 top-left window
    assert tiled[0, 0, 0] == inp[:, :2, :2].sum()


def test_reference_kernel_walk_with_real_weights(built):
    rng = np.random.default_rng(7)
    inp = rng.standard_normal((16, 9, 10)).astype(np.float32)
    k = rng.standard_normal((16, 3, 3, 6)).astype(np.float32)
    assert rel_err(O.ref_tiled(inp, k, 2, 3, 4), O.conv2d_f64(inp[None], k, pad=1, w_layout=O.W_CRSK)[0]) <= FP32_TOL


def test_hand_checkable_stamp(built):
    """One hot pixel stamps the filter flipped: cross-correlation, not convolution; and the
    [k][c][r][s] indexing is told apart from [c][r][s][k]."""
    x = np.zeros((1, 2, 5, 5), np.float32); x[0, 1, 2, 2] = 1.0
    w = np.arange(3 * 2 * 9, dtype=np.float32).reshape(3, 2, 3, 3)
    y = O.conv2d_f32(x, w, pad=1)
    for k in range(3):
        assert np.array_equal(y[0, k, 1:4, 1:4], w[k, 1, ::-1, ::-1])
