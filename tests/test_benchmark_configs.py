"""The configurations the benchmark quotes, at their full sizes, against fp64 and the reference-made goldens.

bench.py reports TK-ResNet-18 at batch 256, TK-VGG-16 in chunks of 128, the Tucker blocks of the ResNet-50 bottleneck
middles at batch 1 and 32, and runs the fp32 kernels with the tiles of the shipped tables.  Each of those is run here
as bench.py runs it and held to its tier's bar: the fp32 FMA kernels and single layers to 1e-5, whole networks on the
tensor-core tier to NET_TC_TOL (tests/helpers.py says why that tier has a bar of its own)."""
import glob
import os

import numpy as np
import pytest
import torch

import oracle as O
from helpers import FP32_TOL, GOLDEN, NET_FP32_TOL, NET_TC_TOL, draw_block, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T(built):
    import tdc_b200
    return tdc_b200


def test_resnet18_at_batch_256(T):
    """224x224, batch 256, the "auto" tier the bench times: six sampled images against the same network in fp64 on
    the GPU; then the fp32 tier on the same images; then the reference network's own logits (batch 2 golden)."""
    import bench
    net = T.fill_deterministic(T.tkc_resnet18(precision="auto").eval(), seed=0).cuda()
    x = torch.randn(256, 3, 224, 224, generator=torch.Generator().manual_seed(4001)).cuda()
    sel = [0, 51, 102, 153, 204, 255]
    with torch.no_grad():
        y = net(x)
        y64 = bench.torch_reference_forward(torch, net.double(), x[sel].double())
        net.float()
        assert rel_err(y[sel].cpu().numpy(), y64.cpu().numpy()) <= NET_TC_TOL
        assert (y[sel].argmax(1) == y64.argmax(1)).all()
        y32 = net.set_precision("fp32")(x[sel].contiguous())
        assert rel_err(y32.cpu().numpy(), y64.cpu().numpy()) <= NET_FP32_TOL
        Z = np.load(os.path.join(GOLDEN, "tk_resnet18.npz"))
        x2 = torch.randn(2, 3, 224, 224, generator=torch.Generator().manual_seed(4001)).cuda()
        assert rel_err(net.set_precision("auto")(x2).cpu().numpy(), Z["logits"]) <= NET_TC_TOL
    from tdc_b200 import tc
    assert tc.status() == 0


def test_vgg16_chunk_of_128(T):
    """224x224, the chunk of 128 images the batch-2048 job is made of, "auto" tier: four sampled images against fp64."""
    import bench
    net = T.tkc_vgg16(precision="auto").eval().cuda()
    x = torch.randn(128, 3, 224, 224, generator=torch.Generator().manual_seed(5001)).cuda()
    sel = [0, 42, 85, 127]
    with torch.no_grad():
        y = net(x)
        y64 = bench.torch_forward_double(torch, net, x[sel])
        assert rel_err(y[sel].cpu().numpy(), y64.cpu().numpy()) <= NET_TC_TOL
        net.precision = "fp32"
        y32 = net(x[sel].contiguous())
        assert rel_err(y32.cpu().numpy(), y64.cpu().numpy()) <= NET_FP32_TOL


@pytest.mark.parametrize("i,Cc,H", [(0, 64, 56), (1, 128, 28), (2, 256, 14), (3, 512, 7)])
@pytest.mark.parametrize("B", [1, 32])
def test_tucker_blocks_of_the_bottleneck_middles(T, i, Cc, H, B):
    """1x1 C->R, 3x3 R->R, 1x1 R->C with R = C/2: the module on every tier against the fp64 chain, as one layer
    (three launches): the single-layer bar."""
    R = Cc // 2
    x, first, core, last, _ = draw_block(3000 + i, B, Cc, Cc, R, R, H, H)

    class HP:
        ranks = {"b": [R, R]}
    m = T.TKConv2dC_B200(Cc, Cc, 3, padding=1, bias=False, hp_dict=HP, name="b")
    with torch.no_grad():
        m.first_kernel.copy_(first); m.core_kernel.copy_(core); m.last_kernel.copy_(last)
    m = m.cuda()
    F = torch.nn.functional
    xd = x.cuda()
    ref = F.conv2d(F.conv2d(F.conv2d(xd.double(), first.cuda().double()), core.cuda().double(), None, 1, 1), last.cuda().double())
    from tdc_b200.dispatch import tucker_strategy
    assert tucker_strategy(m, xd, "auto") == "dense" and tucker_strategy(m, xd, "fp16x3") == "chain"
    with torch.no_grad():
        for precision in ("fp32", "auto", "fp16x3", "tf32x3"):          # "auto": one launch on the merged filter; the others: three
            m.precision = precision
            assert rel_err(m(xd).cpu().numpy(), ref.cpu().numpy()) <= FP32_TOL, precision


def _table_rows():
    from tdc_b200 import tiles
    here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ppopp23-tdc_b200", "tdc_b200", "tables")
    rows = []
    for path in sorted(glob.glob(os.path.join(here, "b200_core3x3_*.csv")) + glob.glob(os.path.join(here, "b200_resnet18_*.csv"))):
        for r in tiles.read_rows(path):
            rows.append((os.path.basename(path), r))
    return rows


def test_every_table_tile_of_the_benchmarked_layers_is_exact(T):
    """The tiles bench.py takes from the shipped tables (the sweep at batch 1 and 64, every conv of TK-ResNet-18 at
    batch 1 and 256), each run on the reference drivers' own check — integers 0..9, all-ones weights, L1 difference 0
    — and, on seeded real-valued data, bit for bit against the oracle that sums in the kernel's order."""
    from tdc_b200._lib import Tile
    rows = _table_rows()
    assert len(rows) >= 50
    for name, r in rows:
        Cc, N, H, W, B, R, stride = (int(r[k]) for k in ("C", "N", "H", "W", "B", "R", "stride"))
        pad = (R - 1) // 2
        tile = Tile(*(int(r[k]) for k in ("th", "tw", "tc", "tn", "nog", "gy", "gx", "imgs", "ks", "kc")))
        nb = min(B, 4)                        # the tile was measured at batch B; its arithmetic does not depend on the batch
        g = torch.Generator().manual_seed(Cc + N + H)
        xi = torch.randint(0, 10, (nb, Cc, H, W), generator=g).float()
        y = T.core_conv2d(xi.cuda(), torch.ones(Cc, R, R, N).cuda(), stride, pad, w_layout=T.W_CRSK, tile=tile)
        exact = O.conv2d_f64(xi.numpy(), np.ones((N, Cc, R, R), np.float32), pad=pad, stride=stride)
        assert np.array_equal(y.cpu().numpy().astype(np.float64), exact), (name, r)
        if Cc * N * H * W * R * R <= 64 * 64 * 28 * 28 * 9:          # the ordered CPU twin is a scalar loop: the smaller layers
            x = torch.randn(1, Cc, H, W, generator=g)
            w = torch.randn(N, Cc, R, R, generator=g) * 0.1
            crsk = w.permute(1, 2, 3, 0).contiguous()
            y = T.core_conv2d(x.cuda(), crsk.cuda(), stride, pad, w_layout=T.W_CRSK, tile=tile).cpu().numpy()
            twin = O.conv2d_f32_sliced(x.numpy(), w.numpy(), pad=pad, stride=stride, tc=tile.tc, ks=tile.ks, kc=tile.kc)
            assert np.array_equal(y, twin), (name, r)


def test_output_that_is_not_16_byte_aligned(T):
    """y offset by one float inside a larger buffer: the fp32 kernel must take its element-wise store path and give
    the very bits of the aligned call (a 16-byte store to such an address would fault)."""
    from tdc_b200 import _lib
    import ctypes as C
    g = torch.Generator().manual_seed(77)
    x = torch.randn(2, 16, 12, 12, generator=g).cuda()
    w = (torch.randn(16, 3, 3, 24, generator=g) * 0.1).cuda()             # [c][r][s][k]
    y = T.core_conv2d(x, w, 1, 1, w_layout=T.W_CRSK)
    buf = torch.zeros(y.numel() + 8, device="cuda")
    odd = buf[1:1 + y.numel()]
    assert odd.data_ptr() % 16 == 4
    rc = T.lib.tdc_core_conv2d_f32(C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(odd.data_ptr()), 2, 16, 12, 12, 24,
                                   3, 3, 1, 1, _lib.W_CRSK, None, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(odd.view_as(y), y) and float(buf[0]) == 0.0 and float(buf[1 + y.numel()]) == 0.0
