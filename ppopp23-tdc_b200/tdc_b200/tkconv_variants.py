"""The reference's other two Tucker modules on the B200 kernels.

* TKConv2dM_B200 — inference/TKConv.py:144-219 (TKConv2dM): factors stored as matrices
  (`first_factor [R1,C]`, `last_factor [K,R2]`) and applied with F.linear on NHWC views there;
  the arithmetic is the same 1x1 -> core -> 1x1 chain, so the forward is the same kernel chain.
* TKConv2dR_B200 — inference/TKConv.py:222-322 (TKConv2dR): rebuilds the dense filter
  W[k,c,r,s] = sum_{a,b} core[a,b,r,s] * last[k,a] * first[b,c] (tensorly's tucker_to_tensor,
  :310) and runs ONE dense convolution.  The rebuild is a weight-load step (einsum, cached until
  a factor changes); only 'zeros' padding is built.

Parameter names and shapes are the reference's, so state dicts interchange.
"""
import math

import torch
import torch.nn as nn
from torch.nn import Parameter, init
from torch.nn.modules.utils import _pair

from . import ops
from ._lib import ERR_UNSUPPORTED, TdcError
from .tkconv import TKConv2dC_B200


class TKConv2dM_B200(nn.Module):
    precision = "fp32"

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode='zeros', hp_dict=None, name=None, dense_w=None, dense_b=None):
        super().__init__()
        if groups != 1:
            raise ValueError("groups must be 1 in this mode")
        if padding_mode != 'zeros':
            raise ValueError("padding_mode must be zero in this mode")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.ranks = hp_dict.ranks[name]
        self.in_rank, self.out_rank = self.ranks[1], self.ranks[0]
        self.kernel_size, self.stride = _pair(kernel_size), _pair(stride)
        self.padding, self.dilation = _pair(padding), _pair(dilation)
        self.groups, self.padding_mode = groups, padding_mode
        self.first_factor = Parameter(torch.empty(self.in_rank, in_channels))
        self.core_kernel = Parameter(torch.empty(self.out_rank, self.in_rank, *self.kernel_size))
        self.last_factor = Parameter(torch.empty(out_channels, self.out_rank))
        if bias:
            self.bias = Parameter(torch.zeros(out_channels))
            if dense_b is not None:
                self.bias.data = dense_b
        else:
            self.register_parameter('bias', None)
        if dense_w is not None:
            from .tucker import partial_tucker_hosvd
            core, (last_factor, first_factor) = partial_tucker_hosvd(dense_w, self.ranks)
            self.first_factor.data = first_factor.t().contiguous()
            self.last_factor.data = last_factor.contiguous()
            self.core_kernel.data = core.contiguous()
        else:
            self.reset_parameters()
        self._core_crsk = None
        self._workspace = None

    def reset_parameters(self):
        init.xavier_uniform_(self.first_factor)
        init.xavier_uniform_(self.last_factor)
        init.xavier_uniform_(self.core_kernel)

    # input checks, the channel-last copy of the core filter and the workspace are those of the C variant
    _check = TKConv2dC_B200._check
    _core_channel_last = TKConv2dC_B200._core_channel_last
    _ws = TKConv2dC_B200._ws

    def forward(self, x):
        x = self._check(x)
        from ._lib import W_CRSK
        return ops.tk_block(x, self.first_factor.detach().view(self.in_rank, self.in_channels, 1, 1),
                            self._core_channel_last(),
                            self.last_factor.detach().view(self.out_channels, self.out_rank, 1, 1),
                            None if self.bias is None else self.bias.detach(), self.stride, self.padding,
                            core_layout=W_CRSK, workspace=self._ws(x))


class TKConv2dR_B200(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode='zeros', hp_dict=None, name=None, dense_w=None, dense_b=None):
        super().__init__()
        if groups != 1 or padding_mode != 'zeros':
            raise TdcError(ERR_UNSUPPORTED, "groups=1 and padding_mode='zeros' are built")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.ranks = list(hp_dict.ranks[name])
        self.in_rank, self.out_rank = self.ranks[1], self.ranks[0]
        self.kernel_size, self.stride = _pair(kernel_size), _pair(stride)
        self.padding, self.dilation = _pair(padding), _pair(dilation)
        self.groups, self.padding_mode = groups, padding_mode
        self.first_factor = Parameter(torch.empty(self.in_rank, in_channels))
        self.core_tensor = Parameter(torch.empty(self.out_rank, self.in_rank, *self.kernel_size))
        self.last_factor = Parameter(torch.empty(out_channels, self.out_rank))
        if bias:
            self.bias = Parameter(torch.zeros(out_channels))
            if dense_b is not None:
                self.bias.data = dense_b
        else:
            self.register_parameter('bias', None)
        if dense_w is not None:
            from .tucker import partial_tucker_hosvd
            core, (last_factor, first_factor) = partial_tucker_hosvd(dense_w, self.ranks)
            self.first_factor.data = first_factor.t().contiguous()
            self.last_factor.data = last_factor.contiguous()
            self.core_tensor.data = core.contiguous()
        else:
            self.reset_parameters()
        self._dense = None

    def reset_parameters(self):
        init.xavier_uniform_(self.first_factor)
        init.xavier_uniform_(self.core_tensor)
        init.xavier_uniform_(self.last_factor)
        if self.bias is not None:
            fan_in = self.in_channels * self.kernel_size[0] * self.kernel_size[1]
            bound = 1 / math.sqrt(fan_in)
            init.uniform_(self.bias, -bound, bound)

    def _recover_weight(self):
        key = tuple((t._version, t.data_ptr()) for t in (self.core_tensor, self.last_factor, self.first_factor))
        if self._dense is None or self._dense[0] != key:
            with torch.no_grad():
                w = torch.einsum("abrs,ka,bc->kcrs", self.core_tensor.double(), self.last_factor.double(),
                                 self.first_factor.double()).float().contiguous()
            self._dense = (key, w)
        return self._dense[1]

    def forward(self, x):
        if self.dilation != (1, 1):
            raise TdcError(ERR_UNSUPPORTED, "dilation %r is not built" % (self.dilation,))
        if not x.is_cuda:
            raise TdcError(ERR_UNSUPPORTED, "TKConv2dR_B200 runs on CUDA tensors only")
        return ops.conv2d(x.contiguous().float(), self._recover_weight(), None if self.bias is None else self.bias.detach(),
                          self.stride, self.padding)
