"""The pooling layer of the end-to-end skeleton (tdc_pool2d_f32) against torch's CPU pooling on the same
seeded input: bit-exact for max (a selection), 1e-6 for averages (summation order)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F


@pytest.fixture(scope="module")
def T(built):
    import tdc_b200
    return tdc_b200


@pytest.mark.gpu
@pytest.mark.parametrize("B,C,H,W,k,s,p", [(2, 3, 16, 16, 3, 2, 1), (3, 5, 112, 112, 3, 2, 1), (2, 5, 15, 13, 3, 2, 1), (1, 4, 8, 8, 2, 2, 0),
                                            (2, 2, 9, 24, 3, 2, 1), (3, 5, 56, 56, 2, 2, 0), (2, 3, 6, 24, 2, 2, 0), (1, 2, 7, 8, 2, 2, 0), (1, 1, 1, 1, 1, 1, 0), (2, 3, 7, 7, 7, 1, 0), (1, 2, 10, 10, 3, 1, 1)])
def test_pooling_matches_torch(T, B, C, H, W, k, s, p):
    x = torch.randn(B, C, H, W, generator=torch.Generator().manual_seed(H * W + k))
    xd = x.cuda()
    assert torch.equal(T.pool2d(xd, k, s, p).cpu(), F.max_pool2d(x, k, s, p))
    inc = T.pool2d(xd, k, s, p, mode=T.ops.POOL_AVG_INCLUDE_PAD).cpu()
    exc = T.pool2d(xd, k, s, p, mode=T.ops.POOL_AVG_EXCLUDE_PAD).cpu()
    assert np.allclose(inc.numpy(), F.avg_pool2d(x, k, s, p, count_include_pad=True).numpy(), rtol=1e-6, atol=1e-6)
    assert np.allclose(exc.numpy(), F.avg_pool2d(x, k, s, p, count_include_pad=False).numpy(), rtol=1e-6, atol=1e-6)


@pytest.mark.gpu
def test_pooling_rejects_bad_windows(T):
    x = torch.zeros(1, 1, 4, 4).cuda()
    for k, s, p in ((3, 1, 2), (5, 1, 0), (0, 1, 0)):
        with pytest.raises(T.TdcError):
            T.pool2d(x, k, s, p)
