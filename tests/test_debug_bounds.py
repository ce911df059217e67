"""The range-checked build of the library (-DTDC_DEBUG_BOUNDS): every global access of the fp32 kernels checks its
offset against its tensor first, and a violation is recorded instead of made.  compute-sanitizer's place in the test
plan: ragged shapes of every kernel family and a whole network run through it, in a process of its own that loads the
variant library, and the record must stay empty while the results stay right."""
import os
import subprocess
import sys

import pytest

from helpers import ROOT

LIB = os.path.join(ROOT, "ppopp23-tdc_b200", "tdc_b200", "libtdc_b200_bounds.so")

CHILD = r'''
import ctypes as C, os, sys
sys.path.insert(0, os.path.join(%(root)r, "ppopp23-tdc_b200"))
import torch
import tdc_b200 as T
assert T.LIB_PATH.endswith("libtdc_b200_bounds.so")
read = T.lib.tdc_debug_bounds_read
read.argtypes = [C.POINTER(C.c_int), C.c_int]
rec = (C.c_int * 4)()
assert read(rec, 1) == 0
F = torch.nn.functional
g = torch.Generator().manual_seed(11)
worst = 0.0
cases = [(1, 3, 5, 1, 1, 1, 1, 0), (2, 7, 9, 2, 3, 3, 1, 1), (5, 33, 130, 9, 13, 3, 1, 1), (3, 20, 40, 15, 13, 3, 2, 1), (2, 16, 24, 9, 9, 5, 1, 2),
         (4, 40, 72, 14, 14, 1, 2, 0), (1, 128, 128, 28, 28, 3, 1, 1), (64, 32, 32, 7, 7, 3, 1, 1), (2, 24, 16, 5, 200, 3, 1, 1), (3, 8, 8, 6, 7, 7, 2, 3),
         (1, 512, 512, 7, 7, 3, 1, 1), (1, 64, 64, 56, 56, 3, 1, 1)]
for (B, Cc, K, H, W, R, stride, pad) in cases:
    x = torch.randn(B, Cc, H, W, generator=g).cuda()
    w = (torch.randn(K, Cc, R, R, generator=g) * 0.1).cuda()
    ref = F.conv2d(x.double(), w.double(), None, stride, pad)
    for wt, layout in ((w, T.W_KCRS), (T.permute_weights(w), T.W_CRSK)):
        y = T.core_conv2d(x, wt, stride, pad, w_layout=layout)
        worst = max(worst, float((y.double() - ref).abs().max() / ref.abs().max()))
    tile = T.best_tile(B, Cc, H, W, K, R, R, pad, stride)
    y = T.core_conv2d(x, T.permute_weights(w), stride, pad, w_layout=T.W_CRSK, tile=tile)
    worst = max(worst, float((y.double() - ref).abs().max() / ref.abs().max()))
net = T.fill_deterministic(T.tkc_resnet18().eval(), 0).cuda()           # "fp32" precision: every conv on the fp32 kernels
with torch.no_grad():
    net(torch.randn(3, 3, 224, 224, generator=g).cuda())
torch.cuda.synchronize()
assert read(rec, 0) == 0
print("BOUNDS", list(rec), "worst", worst)
'''


def test_variant_library_is_built_and_exports_its_record(built):
    import ctypes as C
    assert os.path.exists(LIB)
    assert hasattr(C.CDLL(LIB), "tdc_debug_bounds_read")
    assert not hasattr(C.CDLL(os.path.join(os.path.dirname(LIB), "libtdc_b200.so")), "tdc_debug_bounds_read")


@pytest.mark.gpu
def test_no_access_leaves_its_tensor(built):
    env = dict(os.environ, TDC_B200_LIB=LIB)
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("BOUNDS")][-1]
    rec = eval(line.split("BOUNDS")[1].split("worst")[0])
    assert rec == [0, 0, 0, 0], line
    assert float(line.split("worst")[1]) <= 1e-5
