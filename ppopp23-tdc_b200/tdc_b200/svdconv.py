"""SVD-factorised 1x1 convolutions on libtdc_b200.so — the reference's inference/SVDConv.py.

A 1x1 conv C -> K of rank r is two 1x1 convs, C -> r and r -> K (+ bias).  The three reference classes differ in how
they hold and apply the two factors, not in the result:

* SVDConv2dC (SVDConv.py:122-225): `left_kernel` [r,C,1,1], `right_kernel` [K,r,1,1], two F.conv2d calls;
* SVDConv2dM (:228-296): `left_factor` / `right_factor`, two F.linear calls on the channel-last permutation;
* SVDConv2dR (:16-119): `left_factor` [r,C], `right_factor` [K,r], the dense weight recovered in every forward and
  applied as one conv.  (Its `_recover_weight` multiplies left @ right, which has matching shapes only for
  C == K == r; the product that the factorisation and the other two classes mean is right @ left, and that is what
  is built here.)

Constructor arguments, parameter names and shapes, the ValueErrors for kernel_size / stride / groups / padding_mode,
the xavier-uniform reset and the SVD initialisation from a dense weight (u[:, :r] and diag(s[:r]) @ vt[:r]) are the
reference's, so state dicts load unchanged and the classes can be handed to the reference's model builders.  All of
them run the same two launches of the 1x1 kernels (tensor cores under `precision` != "fp32" where a plan applies);
the bias, and any folded BatchNorm / residual / ReLU a network passes, ride on the second launch.
"""
import torch
import torch.nn as nn
from torch.nn import Parameter, init
from torch.nn.modules.utils import _pair

from ._lib import ERR_UNSUPPORTED, TdcError
from .dispatch import one_conv


def svd_factors(dense_w, rank):
    """(left [r,C], right [K,r]) with right @ left the best rank-r approximation of the [K,C] matrix `dense_w`
    (squeezed from [K,C,1,1]): right = u[:, :r], left = diag(s[:r]) @ vt[:r] — SVDConv.py:175-181.  fp64 SVD,
    rounded once (the reference runs numpy's SVD in the weight's own precision)."""
    m = dense_w.detach().reshape(dense_w.shape[0], dense_w.shape[1]).double().cpu()
    u, s, vt = torch.linalg.svd(m, full_matrices=False)
    right = u[:, :rank].contiguous()
    left = (s[:rank, None] * vt[:rank]).contiguous()
    return left.float(), right.float()


class _SVDConvBase(nn.Module):
    precision = "fp32"
    _names = ("left_kernel", "right_kernel")
    _four_d = True

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode='zeros', hp_dict=None, name=None, dense_w=None, dense_b=None):
        super().__init__()
        kernel_size, stride = _pair(kernel_size), _pair(stride)
        if padding_mode != 'zeros':
            raise ValueError("padding_mode must be zero in this mode")
        if groups != 1:
            raise ValueError("groups must be 1 in this mode")
        if kernel_size[0] * kernel_size[1] != 1:
            raise ValueError('kernel_size must be 1 in this mode')
        if stride[0] * stride[1] != 1:
            raise ValueError('stride must be 1')
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.ranks = hp_dict.ranks[name]
        self.rank = self.ranks if isinstance(self.ranks, int) else self.ranks[0]
        self.kernel_size = kernel_size
        self.stride = stride
        self.padding = _pair(padding)
        self.dilation = _pair(dilation)
        self.transposed = False
        self.output_padding = _pair(0)
        self.groups = groups
        self.padding_mode = padding_mode
        if bias:
            self.bias = Parameter(torch.zeros(out_channels))
            if dense_b is not None:
                self.bias.data = dense_b
        else:
            self.register_parameter('bias', None)
        tail = (1, 1) if self._four_d else ()
        setattr(self, self._names[0], Parameter(torch.empty(self.rank, in_channels, *tail)))
        setattr(self, self._names[1], Parameter(torch.empty(out_channels, self.rank, *tail)))
        if dense_w is not None:
            left, right = svd_factors(dense_w, self.rank)
            getattr(self, self._names[0]).data = left.reshape(self.rank, in_channels, *tail)
            getattr(self, self._names[1]).data = right.reshape(out_channels, self.rank, *tail)
        else:
            self.reset_parameters()

    def reset_parameters(self):
        init.xavier_uniform_(getattr(self, self._names[0]))
        init.xavier_uniform_(getattr(self, self._names[1]))

    def _kernels(self):
        """The two factors as [r,C,1,1] and [K,r,1,1] views of the parameters."""
        left, right = getattr(self, self._names[0]), getattr(self, self._names[1])
        if self._four_d:
            return left, right
        return left.view(self.rank, self.in_channels, 1, 1), right.view(self.out_channels, self.rank, 1, 1)

    def run(self, x, scale=None, shift=None, residual=None, relu=False, precision=None):
        """relu?((right * (left * x) + bias) * scale + shift + residual): the two launches, the epilogue on the
        second."""
        if self.dilation != (1, 1) or self.padding != (0, 0):
            raise TdcError(ERR_UNSUPPORTED, "dilation %r / padding %r are not built for a 1x1 conv" % (self.dilation, self.padding))
        if not x.is_cuda:
            raise TdcError(ERR_UNSUPPORTED, "%s runs on CUDA tensors only" % type(self).__name__)
        if x.dtype != torch.float32 or not x.is_contiguous():
            x = x.contiguous().float()
        p = self.precision if precision is None else precision
        left, right = self._kernels()
        if self.bias is not None:      # (conv + bias) * scale + shift  ->  conv * scale + (bias * scale + shift)
            b = self.bias.detach() if scale is None else self.bias.detach() * scale
            shift = b if shift is None else shift + b
        z = one_conv(self, "left", x, left, None, None, None, None, False, 1, 0, p)
        return one_conv(self, "right", z, right, None, scale, shift, residual, relu, 1, 0, p)

    def forward(self, x):
        return self.run(x)

    def forward_flops(self, x):
        """SVDConv.py:196-216: the output, and MFLOPs of the dense and the factorised conv per image."""
        left, right = self._kernels()
        out = self.run(x)
        height_, width_ = out.shape[2], out.shape[3]
        compr_params = (left.numel() + right.numel()) / 1000
        compr_flops = height_ * width_ * left.numel() / 1000 / 1000 + height_ * width_ * right.numel() / 1000 / 1000
        base_params = self.kernel_size[0] * self.kernel_size[1] * self.in_channels * self.out_channels / 1000
        base_flops = height_ * width_ * self.kernel_size[0] * self.kernel_size[1] * \
            self.in_channels * self.out_channels / 1000 / 1000
        print('baseline # params: {:.2f}K\t compressed # params: {:.2f}K\t '
              'baseline # flops: {:.2f}M\t compressed # flops: {:.2f}M'.format(base_params, compr_params, base_flops,
                                                                               compr_flops))
        return out, base_flops, compr_flops

    def extra_repr(self):
        return ('left_conv(in={}, out={}, kernel_size=(1, 1), bias=False), '
                'right_conv(in={}, out={}, kernel_size={}, stride={}, padding={}, bias={}), '
                .format(self.in_channels, self.rank, self.rank, self.out_channels, self.kernel_size,
                        self.stride, self.padding, self.bias is None))


class SVDConv2dC_B200(_SVDConvBase):
    """inference/SVDConv.py:122-225."""
    _names = ("left_kernel", "right_kernel")
    _four_d = True


class SVDConv2dM_B200(_SVDConvBase):
    """inference/SVDConv.py:228-296 (factors stored [r,C,1,1] / [K,r,1,1] as its constructor allocates them)."""
    _names = ("left_factor", "right_factor")
    _four_d = True


class SVDConv2dR_B200(_SVDConvBase):
    """inference/SVDConv.py:16-119: 2-D factors `left_factor` [r,C], `right_factor` [K,r]; the reference recovers
    the dense weight in every forward, here the two factors are applied one after the other."""
    _names = ("left_factor", "right_factor")
    _four_d = False

    def _recover_weight(self):
        """The dense [K,C,1,1] weight the factors stand for."""
        return self.right_factor.mm(self.left_factor).unsqueeze(-1).unsqueeze(-1)
