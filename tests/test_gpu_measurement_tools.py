"""The two measurement tools behind the phase summary of the tensor-core kernel: the standalone microbenchmark of the
per-SM MMA issue and bulk-copy rates (drivers/tc_rates.cu), and the measurement build of the library
(-DTDC_TC_PROFILE=1, `python kernel_bench.py phases`).  Both are checked for what their numbers must satisfy, not for
the numbers themselves."""
import os
import re
import subprocess
import sys

import pytest

from helpers import ROOT

RATES = os.path.join(ROOT, "ppopp23-tdc_b200", "tdc_b200", "tc_rates")
PROFILE_LIB = os.path.join(ROOT, "ppopp23-tdc_b200", "tdc_b200", "libtdc_b200_profile.so")


def test_rates_tool_is_built(built):
    assert os.path.exists(RATES) and os.access(RATES, os.X_OK)


@pytest.mark.gpu
def test_rates_tool_runs_and_the_kernels_issue_pattern_keeps_the_tensor_core_fed(built):
    r = subprocess.run([RATES], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    mma = {}
    for m in re.finditer(r"mma\s+(\w+)\s+patch rows\s+(\d+), image row\s+(\d+),\s+(\d+) cp.async warps beside it: ([\d.]+) clocks", r.stdout):
        mma.setdefault((m.group(1), int(m.group(4))), []).append(float(m.group(5)))
    assert set(k[0] for k in mma) == {"n128", "conv128", "conv64", "loop128"}
    # a 128 x 128 x 16 fp16 MMA cannot take fewer than 64 clocks on one SM; the kernel's loop must stay within a tenth of that
    for key, vals in mma.items():
        assert all(v >= 63.0 for v in vals), (key, vals)
    assert max(mma[("loop128", 0)]) <= 71.0 and max(mma[("loop128", 12)]) <= 75.0
    copies = [float(m.group(1)) for m in re.finditer(r"copy chunk\s+\d+ bytes, \d in flight: ([\d.]+) bytes per clock", r.stdout)]
    assert len(copies) == 6 and all(c > 5.0 for c in copies)


CHILD = r'''
import ctypes as C, os, sys
sys.path.insert(0, os.path.join(%(root)r, "ppopp23-tdc_b200"))
import torch
import tdc_b200 as T
assert T.LIB_PATH.endswith("libtdc_b200_profile.so")
read = T.lib.tdc_tc_profile_read
read.argtypes = [C.POINTER(C.c_ulonglong), C.c_int]
buf = (C.c_ulonglong * 24)()
g = torch.Generator().manual_seed(3)
x = torch.randn(8, 64, 28, 28, generator=g).cuda()
w = (torch.randn(64, 64, 3, 3, generator=g) * 0.05).cuda()
conv = T.TcConv(w, mode=4)
y = conv(x)
ref = torch.nn.functional.conv2d(x.double(), w.double(), None, 1, 1)
err = float((y.double() - ref).abs().max() / ref.abs().max())
torch.cuda.synchronize()
assert read(buf, 1) == 0
conv(x, out=y)
torch.cuda.synchronize()
assert read(buf, 1) == 0
v = list(buf)
print("RESULT", err, v[16], v[17], v[18], v[19], v[20], v[10], v[11])
'''


@pytest.mark.gpu
def test_measurement_build_marks_the_phases_in_order(built):
    if not os.path.exists(PROFILE_LIB):
        pytest.skip("the measurement build is made on demand (build.py: build_profile)")
    env = dict(os.environ, TDC_B200_LIB=PROFILE_LIB)
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")][0].split()
    err = float(line[1])
    setup, first, issuer_done, last, ctas, issue_clocks, stage_uses = (int(t) for t in line[2:])
    assert err < 1e-5                              # the measurement build computes the same convolution
    assert ctas >= 1 and stage_uses >= ctas        # every CTA with a tile issued at least one stage
    assert 0 < setup < first < issuer_done < last  # sums over the same CTAs: the phases come in this order
    assert issue_clocks > 0
