"""torch.ops.tdc.*: the operators exist, carry shape functions (so graphs that contain them can be traced without a
GPU), and on a GPU give exactly what the direct calls give, also under torch.compile."""
import pytest
import torch


def test_operators_are_registered_with_shape_functions(built):
    import tdc_b200  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    assert hasattr(torch.ops.tdc, "core_conv2d") and hasattr(torch.ops.tdc, "tk_block")
    with FakeTensorMode():
        x = torch.empty(4, 32, 56, 56, device="cuda")
        w = torch.empty(48, 32, 3, 3, device="cuda")
        assert tuple(torch.ops.tdc.core_conv2d(x, w, 1, 1).shape) == (4, 48, 56, 56)
        assert tuple(torch.ops.tdc.core_conv2d(x, w, 2, 1).shape) == (4, 48, 28, 28)
        first, last = torch.empty(32, 64, 1, 1, device="cuda"), torch.empty(80, 48, 1, 1, device="cuda")
        xb = torch.empty(4, 64, 56, 56, device="cuda")
        assert tuple(torch.ops.tdc.tk_block(xb, first, w, last, None, 2, 1).shape) == (4, 80, 28, 28)


@pytest.mark.gpu
def test_operators_equal_the_direct_calls(built):
    import tdc_b200 as T
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 16, 14, 14, generator=g).cuda()
    first, core, last = (torch.randn(s, generator=g).cuda() * 0.2 for s in ((8, 16, 1, 1), (12, 8, 3, 3), (24, 12, 1, 1)))
    bias = torch.randn(24, generator=g).cuda()
    z = torch.randn(2, 8, 14, 14, generator=g).cuda()
    assert torch.equal(torch.ops.tdc.core_conv2d(z, core, 1, 1), T.core_conv2d(z, core, 1, 1))
    assert torch.equal(torch.ops.tdc.tk_block(x, first, core, last, bias, 2, 1), T.tk_block(x, first, core, last, bias, 2, 1))

    def f(x):
        return torch.relu(torch.ops.tdc.tk_block(x, first, core, last, bias, 1, 1)) + 1.0
    want = torch.relu(T.tk_block(x, first, core, last, bias, 1, 1)) + 1.0
    got = torch.compile(f, fullgraph=True)(x)            # the operator is an opaque node of the compiled graph
    assert torch.allclose(got, want, atol=0, rtol=0)
