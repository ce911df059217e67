"""The hot path as torch custom operators: `torch.ops.tdc.core_conv2d` and `torch.ops.tdc.tk_block`.

The reference's operator is a torch module whose forward is three F.conv2d calls (inference/TKConv.py:90-95), ops that
torch.compile and torch.export know.  These two operators give the replacement the same standing: each has a shape
function (register_fake), so a graph that contains them can be traced, exported and compiled around them; the
implementation is the C ABI call the module makes anyway (tdc_core_conv2d_f32 / tdc_tk_block_f32 through `ops`).
Inference only: no autograd formula is registered, as the library has no backward kernels.

    y = torch.ops.tdc.core_conv2d(x, w_kcrs, stride, padding)
    y = torch.ops.tdc.tk_block(x, first, core_kcrs, last, bias_or_None, stride, padding)
"""
from typing import Optional

import torch
from torch import Tensor

from . import ops


def _out_hw(H, W, R, S, pad, stride):
    return (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1


@torch.library.custom_op("tdc::core_conv2d", mutates_args=(), device_types="cuda")
def core_conv2d(x: Tensor, w: Tensor, stride: int, padding: int) -> Tensor:
    return ops.core_conv2d(x, w, stride, padding)


@core_conv2d.register_fake
def _(x, w, stride, padding):
    B, _, H, W = x.shape
    K, _, R, S = w.shape
    Ho, Wo = _out_hw(H, W, R, S, padding, stride)
    return x.new_empty((B, K, Ho, Wo))


@torch.library.custom_op("tdc::tk_block", mutates_args=(), device_types="cuda")
def tk_block(x: Tensor, first: Tensor, core: Tensor, last: Tensor, bias: Optional[Tensor], stride: int, padding: int) -> Tensor:
    return ops.tk_block(x, first, core, last, bias, stride, padding)


@tk_block.register_fake
def _(x, first, core, last, bias, stride, padding):
    B, _, H, W = x.shape
    _, _, R, S = core.shape
    Ho, Wo = _out_hw(H, W, R, S, padding, stride)
    return x.new_empty((B, last.shape[0], Ho, Wo))
