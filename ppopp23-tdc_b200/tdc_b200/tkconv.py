"""TKConv2dC_B200 — the reference's Tucker-2 conv module with its forward on libtdc_b200.so.

Mirrors inference/TKConv.py:23-141 (class TKConv2dC): same constructor arguments, same
parameter names and shapes (first_kernel [R1,C,1,1], core_kernel [R2,R1,kh,kw], last_kernel
[K,R2,1,1], bias [K] or None), same ValueError for groups != 1 / padding_mode != 'zeros',
same xavier-uniform reset, same forward_features / forward_flops / extra_repr outputs.  A
state dict saved from the reference module loads unchanged, and the class can be passed as
the `conv=` argument of the reference's model builders (inference/resnet_inet_tt.py:32-38).
"""
from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor
from torch.nn import Parameter, init
from torch.nn.modules.utils import _pair

from . import ops, tiles
from ._lib import W_CRSK, TdcError, ERR_UNSUPPORTED


_SHARED_WS = {}     # device -> uint8 tensor


class TKConv2dC_B200(nn.Module):
    # "fp32": the fp32 FMA kernels (bit-reproducible, summation order documented);
    # "fp16x3" / "tf32x3": tensor cores with operands split into two fp16 / TF32 parts, fp32-level results (1e-5 bar;
    #     fp16 parts need |x| and |w| within fp16's range of 65504);
    # "tf32": tensor cores, plain TF32 (5e-3 bar);
    # "auto": split operands where the layer is large enough to fill the GPU, fp32 otherwise.
    precision = "fp32"

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, bias: bool = True, padding_mode: str = 'zeros', hp_dict: Optional = None,
                 name: str = None, dense_w: Tensor = None, dense_b: Tensor = None):
        if groups != 1:
            raise ValueError("groups must be 1 in this mode")
        if padding_mode != 'zeros':
            raise ValueError("padding_mode must be zero in this mode")
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.ranks = hp_dict.ranks[name]          # [out_rank (R2), in_rank (R1)], TKConv.py:52-54
        self.in_rank = self.ranks[1]
        self.out_rank = self.ranks[0]
        self.kernel_size = _pair(kernel_size)
        self.stride = _pair(stride)
        self.padding = _pair(padding)
        self.dilation = _pair(dilation)
        self.transposed = False
        self.output_padding = _pair(0)
        self.groups = groups
        self.padding_mode = padding_mode

        self.first_kernel = Parameter(torch.empty(self.in_rank, in_channels, 1, 1))
        self.core_kernel = Parameter(torch.empty(self.out_rank, self.in_rank, *self.kernel_size))
        self.last_kernel = Parameter(torch.empty(out_channels, self.out_rank, 1, 1))
        if bias:
            self.bias = Parameter(torch.zeros(out_channels))
            if dense_b is not None:
                self.bias.data = dense_b
        else:
            self.register_parameter('bias', None)
        if dense_w is not None:
            from .tucker import partial_tucker_hosvd
            core, (last_factor, first_factor) = partial_tucker_hosvd(dense_w, self.ranks)
            self.first_kernel.data = first_factor.t().contiguous().unsqueeze(-1).unsqueeze(-1)
            self.last_kernel.data = last_factor.contiguous().unsqueeze(-1).unsqueeze(-1)
            self.core_kernel.data = core.contiguous()
        else:
            self.reset_parameters()
        self._core_crsk = None      # (version, data_ptr, tensor): channel-last copy of core_kernel
        self._workspace = None

    def reset_parameters(self) -> None:
        init.xavier_uniform_(self.first_kernel)
        init.xavier_uniform_(self.core_kernel)
        init.xavier_uniform_(self.last_kernel)

    # -- B200 path ---------------------------------------------------------------------
    def _check(self, x):
        if self.dilation != (1, 1):
            raise TdcError(ERR_UNSUPPORTED, "dilation %r is not built" % (self.dilation,))
        if not x.is_cuda:
            raise TdcError(ERR_UNSUPPORTED, "TKConv2dC_B200 runs on CUDA tensors only")
        return x.contiguous().float() if (x.dtype != torch.float32 or not x.is_contiguous()) else x

    def _core_channel_last(self):
        w = self.core_kernel
        key = (w._version, w.data_ptr())
        if self._core_crsk is None or self._core_crsk[0] != key:
            self._core_crsk = (key, ops.permute_weights(w.detach().contiguous()))
        return self._core_crsk[1]

    def _factor_channel_last(self, name):
        """[C][1][1][K] copy of a 1x1 factor (`first_kernel` / `last_kernel`), rebuilt when the parameter changes."""
        w = getattr(self, name)
        key = (w._version, w.data_ptr())
        store = self.__dict__.setdefault("_factor_crsk", {})
        hit = store.get(name)
        if hit is None or hit[0] != key:
            hit = store[name] = (key, ops.permute_weights(w.detach().contiguous()))
        return hit[1]

    def fold_pays(self):
        """True when the core and the last 1x1 step, multiplied into ONE kh x kw conv R1 -> K, cost no more
        multiply-adds than the two steps apart (K <= R2, roughly: the dense layers of TK-DenseNet, 32 -> 32 -> 32)."""
        rs = self.kernel_size[0] * self.kernel_size[1]
        return rs * self.in_rank * self.out_channels <= rs * self.in_rank * self.out_rank + self.out_rank * self.out_channels

    def _core_last(self):
        """(KCRS, channel-last) copies of last o core: w[k][c][i][j] = sum_r last[k][r] * core[r][c][i][j], summed in
        fp64 and rounded once; rebuilt when either parameter changes.  The same linear map as the two steps, one
        launch and one intermediate fewer; results differ from the two-step chain by fp32 rounding only."""
        key = (self.core_kernel._version, self.core_kernel.data_ptr(), self.last_kernel._version, self.last_kernel.data_ptr())
        hit = self.__dict__.get("_core_last_cache")
        if hit is None or hit[0] != key:
            w = torch.einsum("kr,rcij->kcij", self.last_kernel.detach().double()[:, :, 0, 0], self.core_kernel.detach().double())
            w = w.float().contiguous()
            hit = self.__dict__["_core_last_cache"] = (key, w, ops.permute_weights(w))
        return hit[1], hit[2]

    def _dense_weight(self):
        """The block as ONE kh x kw filter C -> K: w[k][c][i][j] = sum_{r2,r1} last[k][r2] * core[r2][r1][i][j] * first[r1][c],
        summed in fp64 and rounded once; rebuilt when a factor changes.  It is the weight the reference's TKConv2dR
        recovers before its single conv (inference/TKConv.py:310-322): the same linear map as the three steps, with
        no intermediate at all.  It costs 9CK multiply-adds per pixel against C*R1 + 9*R1*R2 + R2*K, and on this GPU
        it is still the faster form whenever the three steps are bound by their launches and memory passes rather
        than by arithmetic (`dispatch.tucker_strategy` decides)."""
        ps = (self.first_kernel, self.core_kernel, self.last_kernel)
        key = tuple((p._version, p.data_ptr()) for p in ps)
        hit = self.__dict__.get("_dense_cache")
        if hit is None or hit[0] != key:
            t = torch.einsum("abij,bc->acij", self.core_kernel.detach().double(), self.first_kernel.detach().double()[:, :, 0, 0])
            w = torch.einsum("ka,acij->kcij", self.last_kernel.detach().double()[:, :, 0, 0], t).float().contiguous()
            hit = self.__dict__["_dense_cache"] = (key, w)
        return hit[1]

    def _ws(self, x, shared=False):
        """Workspace for the block's two intermediates: this module's own, or (shared=True) one
        buffer per device that all blocks of a network reuse — they run one after another on one
        stream, and a small shared buffer stays L2-resident."""
        B, C, H, W = x.shape
        need = ops.tk_block_workspace_bytes(B, C, H, W, self.in_rank, self.out_rank, self.out_channels,
                                            self.kernel_size[0], self.kernel_size[1], self.padding[0], self.stride[0])
        if shared:
            ws = _SHARED_WS.get(x.device)
            if ws is None or ws.numel() < need:
                ws = _SHARED_WS[x.device] = torch.empty(need, device=x.device, dtype=torch.uint8)
            return ws
        ws = self._workspace
        if ws is None or ws.numel() < need or ws.device != x.device:
            ws = self._workspace = torch.empty(need, device=x.device, dtype=torch.uint8)
        return ws

    def forward(self, x):
        x = self._check(x)
        if self.precision != "fp32" and self.stride[0] == self.stride[1] and self.padding[0] == self.padding[1]:
            # each of the three steps on the kernel that suits it (tensor cores where a plan exists and, under
            # "auto", the step is large enough; the fp32 FMA kernel with its table tile otherwise)
            from .dispatch import one_conv, tucker_strategy
            p = self.precision
            bias = None if self.bias is None else self.bias.detach()
            if tucker_strategy(self, x, p) == "dense":
                return one_conv(self, "dense", x, self._dense_weight(), None, None, bias, None, False, self.stride[0], self.padding[0], p)
            z1 = one_conv(self, "first", x, self.first_kernel, lambda: self._factor_channel_last("first_kernel"),
                          None, None, None, False, 1, 0, p)
            z2 = one_conv(self, "core", z1, self.core_kernel, self._core_channel_last, None, None, None, False,
                          self.stride[0], self.padding[0], p)
            return one_conv(self, "last", z2, self.last_kernel, lambda: self._factor_channel_last("last_kernel"),
                            None, bias, None, False, 1, 0, p)
        B, _, H, W = x.shape
        tile = tiles.table_tile(B, self.in_rank, H, W, self.out_rank, self.kernel_size[0], self.kernel_size[1],
                                self.padding[0], self.stride[0])     # measured table first, model otherwise
        bias = None if self.bias is None else self.bias.detach()
        Ho, Wo = ops.out_hw(H, W, self.kernel_size[0], self.kernel_size[1], self.padding[0], self.stride[0])
        t1 = tiles.table_tile(B, self.in_channels, H, W, self.in_rank, 1, 1, 0, 1)
        t3 = tiles.table_tile(B, self.out_rank, Ho, Wo, self.out_channels, 1, 1, 0, 1)
        if t1 is not None or t3 is not None:
            # measured tiles exist for the 1x1 steps: the same three launches, each with its table tile and its
            # channel-last filter copy (tdc_tk_block_f32 takes a tile for the core only)
            z1 = ops.conv2d(x, self._factor_channel_last("first_kernel"), w_layout=W_CRSK, tile=t1)
            z2 = ops.core_conv2d(z1, self._core_channel_last(), self.stride, self.padding, w_layout=W_CRSK, tile=tile)
            return ops.conv2d(z2, self._factor_channel_last("last_kernel"), bias, w_layout=W_CRSK, tile=t3)
        return ops.tk_block(x, self.first_kernel.detach(), self._core_channel_last(), self.last_kernel.detach(),
                            bias, self.stride, self.padding, core_layout=W_CRSK, workspace=self._ws(x), core_tile=tile)

    def forward_features(self, x):
        x = self._check(x)
        features = []
        out = ops.conv2d(x, self.first_kernel.detach())
        features.append(out)
        out = ops.core_conv2d(out, self._core_channel_last(), self.stride, self.padding, w_layout=W_CRSK)
        features.append(out)
        out = ops.conv2d(out, self.last_kernel.detach(), None if self.bias is None else self.bias.detach())
        features.append(out)
        return out, features

    def forward_flops(self, x):
        compr_params = (self.first_kernel.numel() + self.core_kernel.numel() + self.last_kernel.numel()) / 1000
        out, feats = self.forward_features(x)
        compr_flops = 0
        for f, k in zip(feats, (self.first_kernel, self.core_kernel, self.last_kernel)):
            compr_flops += f.shape[2] * f.shape[3] * k.numel() / 1000 / 1000
        height_, width_ = out.shape[2], out.shape[3]
        base_params = self.kernel_size[0] * self.kernel_size[1] * self.in_channels * self.out_channels / 1000
        base_flops = height_ * width_ * self.kernel_size[0] * self.kernel_size[1] * \
            self.in_channels * self.out_channels / 1000 / 1000
        print('baseline # params: {:.2f}K\t compressed # params: {:.2f}K\t '
              'baseline # flops: {:.2f}M\t compressed # flops: {:.2f}M'.format(base_params, compr_params, base_flops,
                                                                               compr_flops))
        return out, base_flops, compr_flops

    def extra_repr(self):
        return ('first_conv(in={}, out={}, kernel_size=(1, 1), bias=False), '
                'core_conv(in={}, out={}, kernel_size={}, stride={}, padding={}, bias={}), '
                'last_conv(in={}, out={}, kernel_size=(1, 1), bias=False)'
                .format(self.in_channels, self.in_rank, self.in_rank, self.out_rank, self.kernel_size,
                        self.stride, self.padding, self.bias is None, self.out_rank, self.out_channels))
