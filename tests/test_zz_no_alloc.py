"""The no-allocation Tucker block (tdc_tk_block_f32_static) against the regular entry point.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.  The entry point exists for callers that cannot allocate device memory
— a serving loop with a fixed arena, a plug-in inside a framework that owns the allocator —
so the test hands it nothing but inputs and outputs and checks that two calls in a row, which
share the library's built-in workspace and find the previous call's data in it, each give what
tdc_tk_block_f32 gives with a caller-provided workspace.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import FP32_TOL, draw_block, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T(built):
    import tdc_b200
    assert torch.cuda.is_available()
    return tdc_b200


def run_both(T, seed, B, Cc, K, R1, R2, H, W, k, stride, pad, bias):
    from tdc_b200 import _lib
    x, first, core, last, b = draw_block(seed, B, Cc, K, R1, R2, H, W, k, bias)
    xd, fd, cd, ld = x.cuda(), first.cuda(), core.cuda(), last.cuda()
    bd = b.cuda() if b is not None else None
    Ho, Wo = T.out_hw(H, W, k, k, pad, stride)
    ref = T.tk_block(xd, fd, cd, ld, bd, stride, pad)                       # existing entry point
    y = torch.full((B, K, Ho, Wo), float("nan"), device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    rc = T.lib.tdc_tk_block_f32_static(ptr(xd), ptr(fd), ptr(cd), ptr(ld), ptr(bd), ptr(y), B, Cc, H, W, R1, R2, K, k, k,
                                       pad, stride, _lib.W_KCRS, _lib.EPI_NONE, None,
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, T.lib.tdc_last_error_string()
    torch.cuda.synchronize()
    return y.cpu().numpy(), ref.cpu().numpy()


def test_two_calls_in_a_row_match_the_regular_entry_point(T):
    # first call: sets up the workspace address for this device and fills the workspace
    y1, r1 = run_both(T, 501, 4, 32, 48, 16, 24, 28, 28, 3, 1, 1, True)
    assert rel_err(y1, r1) <= FP32_TOL and np.array_equal(y1, r1)
    # second call: another shape and stride, so it finds the first call's data where its own
    # intermediates go; nothing of it may show in the result
    y2, r2 = run_both(T, 502, 2, 24, 40, 12, 20, 14, 14, 3, 2, 1, False)
    assert rel_err(y2, r2) <= FP32_TOL and np.array_equal(y2, r2)
    # and the first problem again gives the first answer again
    y3, _ = run_both(T, 501, 4, 32, 48, 16, 24, 28, 28, 3, 1, 1, True)
    assert np.array_equal(y3, y1)


def test_the_call_itself_claims_no_device_memory(T):
    """The property the entry point exists for, measured: with every buffer of the call allocated beforehand, free
    device memory as the driver reports it (cudaMemGetInfo, which sees every allocation of the process, cached or not)
    is the same before and after a second and a third call.  (The first call on a device may load the library's code,
    built-in workspace included; that is the start-up call the header asks for.)"""
    from tdc_b200 import _lib
    x, first, core, last, b = draw_block(503, 4, 32, 48, 16, 24, 28, 28, 3, True)
    xd, fd, cd, ld, bd = x.cuda(), first.cuda(), core.cuda(), last.cuda(), b.cuda()
    y = torch.empty(4, 48, 28, 28, device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr())
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        rc = T.lib.tdc_tk_block_f32_static(ptr(xd), ptr(fd), ptr(cd), ptr(ld), ptr(bd), ptr(y), 4, 32, 28, 28, 16, 24, 48, 3, 3,
                                           1, 1, _lib.W_KCRS, _lib.EPI_NONE, None, st)
        torch.cuda.synchronize()
        return rc
    assert call() == 0                                   # start-up call
    free0 = torch.cuda.mem_get_info()[0]
    assert call() == 0
    free1 = torch.cuda.mem_get_info()[0]
    assert call() == 0
    free2 = torch.cuda.mem_get_info()[0]
    assert free0 == free1 == free2
    # a missing input is refused with a status code, nothing is dereferenced
    rc = T.lib.tdc_tk_block_f32_static(None, ptr(fd), ptr(cd), ptr(ld), ptr(bd), ptr(y), 4, 32, 28, 28, 16, 24, 48, 3, 3,
                                       1, 1, _lib.W_KCRS, _lib.EPI_NONE, None, st)
    assert rc == _lib.ERR_NULL and T.lib.tdc_last_error_string()


def test_sizes_beyond_the_built_in_workspace_are_rejected(T):
    from tdc_b200 import _lib
    B, Cc, R1, R2, K, H = 64, 64, 32, 32, 64, 56            # needs 51 MB of intermediates
    assert T.tk_block_workspace_bytes(B, Cc, H, H, R1, R2, K, 3, 3, 1, 1) > _lib.STATIC_WORKSPACE_BYTES
    d = torch.zeros(8, device="cuda")
    p = C.c_void_p(d.data_ptr())                               # never dereferenced: the size check comes first
    rc = T.lib.tdc_tk_block_f32_static(p, p, p, p, None, p, B, Cc, H, H, R1, R2, K, 3, 3, 1, 1, _lib.W_KCRS,
                                       _lib.EPI_NONE, None, None)
    assert rc == _lib.ERR_WORKSPACE
    msg = T.lib.tdc_last_error_string().decode()
    assert str(_lib.STATIC_WORKSPACE_BYTES) in msg and "tdc_tk_block_f32" in msg
