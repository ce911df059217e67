"""TK-compressed DenseNet-BC on the B200 kernels — the assembly of the reference's TenDenseNet.

Mirrors inference/densenet_inet_tt.py: TenDenseLayer (:36-117), TenDenseBlock (:120-139), TenDenseTransition
(:142-159), TenDenseNet (:162-281) and the `tkc_densenet121/201/264` entries (:315-364), in the default configuration
(7x7 stem, no anti-aliasing layer, no dropout, no checkpointing).  Module names, parameter names and shapes are the
reference's, so a state dict of `TenDenseNet(conv=TKConv2dC, hp_dict=...)` loads unchanged.  As there, a layer's 1x1
bottleneck conv is an SVD conv and its 3x3 conv a Tucker conv when their keys are in `hp_dict.ranks`; the shipped
dictionaries (inference/hp_dicts/tk_densenet121_hp.py:126-) list only the 3x3 convs, with ranks [32, 32].

What runs where (eval mode only):

* a dense block keeps ONE feature buffer [B][C0 + n*growth][H][W]; layer i reads its first C0 + i*growth channels in
  place and appends its `growth` new ones, so nothing is concatenated again (the reference's torch.cat per layer,
  :58-60, re-copies every earlier feature; Concate::forward of the C++ skeleton likewise);
* norm1 + ReLU (timm's BatchNormAct2d: BatchNorm2d followed by ReLU) is one strided scale/shift/ReLU launch over that
  prefix; norm2 + ReLU is folded into the last launch of conv1; conv2 writes its features, which one strided copy
  launch appends to the buffer.  Outside "fp32" precision a Tucker conv2 whose last 1x1 step is no wider than its
  core (32 -> 32 here) runs as two launches, the last factor multiplied into the core filter once;
* a transition is scale/shift/ReLU, the 1x1 conv, and the 2x2 average pool of the pooling kernel;
* the stem folds norm0 + ReLU into the 7x7 conv's launch; global average pool and classifier stay torch ops.
"""
from collections import OrderedDict

import torch
import torch.nn as nn

from . import ops
from ._lib import ERR_UNSUPPORTED, TdcError
from .dispatch import one_conv as _one_conv, tucker_strategy
from .resnet import Conv2dB200, _fold_bn, _tk_or_dense
from .svdconv import SVDConv2dC_B200
from .tkconv import TKConv2dC_B200


class BatchNormReLU2d(nn.BatchNorm2d):
    """BatchNorm2d followed by ReLU under the parameter names of BatchNorm2d — what timm's BatchNormAct2d, the
    reference's `norm_layer` default (densenet_inet_tt.py:18,37,178), is with its default activation.  The eager
    forward below is for CPU checks; the network folds it into kernels."""

    def forward(self, x):
        return torch.relu(super().forward(x))


class Growth32Ranks:
    """hp_dict in the form of inference/hp_dicts/tk_densenet121_hp.py:126-: every 3x3 conv of every dense layer
    (`features.denseblock{s}.denselayer{i}.conv2.weight`, bn_size*growth -> growth) Tucker with ranks
    [R2, R1] = [growth, growth]; the 1x1 convs stay dense."""

    def __init__(self, block_config=(6, 12, 24, 16), growth_rate=32):
        self.ranks = {}
        for s, n in enumerate(block_config, start=1):
            for i in range(1, n + 1):
                self.ranks["features.denseblock%d.denselayer%d.conv2.weight" % (s, i)] = [growth_rate, growth_rate]


def _conv(module, x, scale, shift, relu, precision):
    if isinstance(module, SVDConv2dC_B200):
        return module.run(x, scale, shift, None, relu, precision)
    if isinstance(module, TKConv2dC_B200) and precision != "fp32" and module.fold_pays() and tucker_strategy(module, x, precision) != "dense":
        # 128 -> 32 -> 32 -> 32: the last 1x1 step multiplied into the core filter — two launches instead of three
        # ("fp32" keeps the reference's three-step chain)
        if module.bias is not None:
            b = module.bias.detach() if scale is None else module.bias.detach() * scale
            shift = b if shift is None else shift + b
        z = _one_conv(module, "first", x, module.first_kernel, lambda: module._factor_channel_last("first_kernel"),
                      None, None, None, False, 1, 0, precision)
        w, w_cl = module._core_last()
        return _one_conv(module, "core_last", z, w, w_cl, scale, shift, None, relu, module.stride[0], module.padding[0], precision)
    return _tk_or_dense(module, x, scale, shift, None, relu, precision)


class TKDenseLayer(nn.Module):
    """densenet_inet_tt.py:36-117."""

    def __init__(self, num_input_features, growth_rate, bn_size, stage=None, id=None, hp_dict=None, dense_dict=None):
        super().__init__()
        self.norm1 = BatchNormReLU2d(num_input_features)
        mid = bn_size * growth_rate
        w_name = "features.denseblock%s.denselayer%s.conv1.weight" % (stage, id)
        if w_name in hp_dict.ranks:
            self.conv1 = SVDConv2dC_B200(num_input_features, mid, kernel_size=1, stride=1, bias=False, hp_dict=hp_dict,
                                         name=w_name, dense_w=None if not dense_dict else dense_dict[w_name])
        else:
            self.conv1 = Conv2dB200(num_input_features, mid, kernel_size=1, stride=1, bias=False)
        self.norm2 = BatchNormReLU2d(mid)
        w_name = "features.denseblock%s.denselayer%s.conv2.weight" % (stage, id)
        if w_name in hp_dict.ranks:
            self.conv2 = TKConv2dC_B200(mid, growth_rate, kernel_size=3, stride=1, padding=1, bias=False, hp_dict=hp_dict,
                                        name=w_name, dense_w=None if not dense_dict else dense_dict[w_name])
        else:
            self.conv2 = Conv2dB200(mid, growth_rate, kernel_size=3, stride=1, padding=1, bias=False)
        self.num_input_features = num_input_features
        self.growth_rate = growth_rate

    def new_features(self, prefix, precision):
        """`prefix`: the first num_input_features channels of the block's buffer (a view).  Returns the layer's
        `growth_rate` new feature maps."""
        s1, b1 = _fold_bn(self.norm1)
        s2, b2 = _fold_bn(self.norm2)
        a = ops.affine_relu(prefix, s1, b1, relu=True)
        z = _conv(self.conv1, a, s2, b2, True, precision)
        return _conv(self.conv2, z, None, None, False, precision)

    def forward(self, x):
        feats = torch.cat(x, 1) if isinstance(x, (list, tuple)) else x
        return self.new_features(feats.contiguous(), getattr(self, "precision", "fp32"))


class TKDenseBlock(nn.ModuleDict):
    """densenet_inet_tt.py:120-139, on one feature buffer."""

    def __init__(self, num_layers, num_input_features, bn_size, growth_rate, stage=None, hp_dict=None, dense_dict=None):
        super().__init__()
        for i in range(num_layers):
            self.add_module("denselayer%d" % (i + 1),
                            TKDenseLayer(num_input_features + i * growth_rate, growth_rate, bn_size, stage=stage, id=i + 1,
                                         hp_dict=hp_dict, dense_dict=dense_dict))
        self.num_input_features = num_input_features
        self.num_output_features = num_input_features + num_layers * growth_rate

    def forward(self, init_features):
        B, C0, H, W = init_features.shape
        buf = torch.empty((B, self.num_output_features, H, W), device=init_features.device, dtype=torch.float32)
        ops.affine_relu(init_features, None, None, relu=False, out=buf[:, :C0])
        c = C0
        precision = getattr(self, "precision", "fp32")
        for layer in self.values():
            y = layer.new_features(buf[:, :c], precision)
            ops.affine_relu(y, None, None, relu=False, out=buf[:, c:c + y.shape[1]])
            c += y.shape[1]
        return buf


class TKDenseTransition(nn.Sequential):
    """densenet_inet_tt.py:142-159 (norm, conv, 2x2 average pool)."""

    def __init__(self, num_input_features, num_output_features, stage=None, hp_dict=None, dense_dict=None):
        super().__init__()
        self.add_module("norm", BatchNormReLU2d(num_input_features))
        w_name = "features.transition%s.conv.weight" % stage
        if w_name in hp_dict.ranks:
            self.add_module("conv", SVDConv2dC_B200(num_input_features, num_output_features, kernel_size=1, stride=1, bias=False,
                                                    hp_dict=hp_dict, name=w_name,
                                                    dense_w=None if dense_dict is None else dense_dict[w_name]))
        else:
            self.add_module("conv", Conv2dB200(num_input_features, num_output_features, kernel_size=1, stride=1, bias=False))
        self.add_module("pool", nn.AvgPool2d(kernel_size=2, stride=2))

    def forward(self, x):
        s, b = _fold_bn(self.norm)
        a = ops.affine_relu(x, s, b, relu=True)
        z = _conv(self.conv, a, None, None, False, getattr(self, "precision", "fp32"))
        return ops.pool2d(z, self.pool.kernel_size, self.pool.stride, self.pool.padding, mode=ops.POOL_AVG_INCLUDE_PAD)


class TKDenseNet(nn.Module):
    """densenet_inet_tt.py:162-281 (TenDenseNet) in its default configuration."""

    def __init__(self, growth_rate=32, block_config=(6, 12, 24, 16), bn_size=4, num_classes=1000, in_chans=3,
                 hp_dict=None, dense_dict=None, precision="fp32"):
        super().__init__()
        if hp_dict is None:
            hp_dict = Growth32Ranks(block_config, growth_rate)
        self.num_classes = num_classes
        num_init_features = growth_rate * 2
        self.features = nn.Sequential(OrderedDict([
            ("conv0", Conv2dB200(in_chans, num_init_features, kernel_size=7, stride=2, padding=3, bias=False)),
            ("norm0", BatchNormReLU2d(num_init_features)),
            ("pool0", nn.MaxPool2d(kernel_size=3, stride=2, padding=1)),
        ]))
        num_features = num_init_features
        for i, num_layers in enumerate(block_config):
            block = TKDenseBlock(num_layers, num_features, bn_size, growth_rate, stage=i + 1, hp_dict=hp_dict, dense_dict=dense_dict)
            self.features.add_module("denseblock%d" % (i + 1), block)
            num_features = num_features + num_layers * growth_rate
            if i != len(block_config) - 1:
                self.features.add_module("transition%d" % (i + 1),
                                         TKDenseTransition(num_features, num_features // 2, stage=i + 1, hp_dict=hp_dict,
                                                           dense_dict=dense_dict))
                num_features = num_features // 2
        self.features.add_module("norm5", BatchNormReLU2d(num_features))
        self.num_features = num_features
        self.global_pool = nn.AdaptiveAvgPool2d(1)          # timm's create_classifier(pool_type='avg'): pool, flatten, Linear
        self.classifier = nn.Linear(num_features, num_classes)
        for m in self.modules():                            # the reference's init loop, :256-263
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight)
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.Linear):
                nn.init.constant_(m.bias, 0)
        self.set_precision(precision)

    def set_precision(self, precision):
        """"fp32": every conv on the fp32 FMA kernels; "auto": large layers on tensor cores with split operands
        (fp32-level results); "tf32x3" / "tf32": every conv with a tensor-core plan on tensor cores."""
        if precision not in ("fp32", "auto", "fp16x3", "tf32x3", "tf32"):
            raise ValueError("precision %r" % (precision,))
        self.precision = precision
        for m in self.modules():
            if isinstance(m, (TKDenseLayer, TKDenseBlock, TKDenseTransition)):
                m.precision = precision
        return self

    def get_classifier(self):
        return self.classifier

    def forward_features(self, x):
        if self.training:
            raise TdcError(ERR_UNSUPPORTED, "training-mode BatchNorm is not built; call .eval()")
        if not x.is_cuda:
            raise TdcError(ERR_UNSUPPORTED, "TKDenseNet runs on CUDA tensors only")
        f = self.features
        x = x.contiguous().float()
        s, b = _fold_bn(f.norm0)
        x = _tk_or_dense(f.conv0, x, s, b, None, True, self.precision)
        x = ops.pool2d(x, f.pool0.kernel_size, f.pool0.stride, f.pool0.padding)
        for name, m in f.named_children():
            if name.startswith(("denseblock", "transition")):
                x = m(x)
        s, b = _fold_bn(f.norm5)
        return ops.affine_relu(x, s, b, relu=True)

    def forward(self, x):
        x = self.forward_features(x)
        return self.classifier(torch.flatten(self.global_pool(x), 1))


def tkc_densenet121(hp_dict=None, num_classes=1000, precision="fp32", dense_dict=None):
    """densenet_inet_tt.py:315-330 without the checkpoint load: growth 32, blocks (6, 12, 24, 16)."""
    return TKDenseNet(32, (6, 12, 24, 16), num_classes=num_classes, hp_dict=hp_dict, dense_dict=dense_dict, precision=precision)


def tkc_densenet201(hp_dict=None, num_classes=1000, precision="fp32", dense_dict=None):
    """densenet_inet_tt.py:349-364: growth 32, blocks (6, 12, 48, 32)."""
    return TKDenseNet(32, (6, 12, 48, 32), num_classes=num_classes, hp_dict=hp_dict, dense_dict=dense_dict, precision=precision)


def tkc_densenet264(hp_dict=None, num_classes=1000, precision="fp32", dense_dict=None):
    """densenet_inet_tt.py:332-347: growth 48, blocks (6, 12, 64, 48)."""
    return TKDenseNet(48, (6, 12, 64, 48), num_classes=num_classes, hp_dict=hp_dict, dense_dict=dense_dict, precision=precision)
