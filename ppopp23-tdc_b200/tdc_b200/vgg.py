"""TK-compressed VGG on the B200 kernels — the feature stack of the reference's TenVGG.

Mirrors inference/vgg_tt.py:44-49 (cfgs) and :90-136 (TenVGG.__init__, the `features`
Sequential): 3x3 convs with padding 1 and a bias, a Tucker conv wherever
`features.{id}.weight` is in `hp_dict.ranks` (id counts conv/[norm]/act modules, so the
state-dict keys are the reference's), 2x2 max-pools at the 'M' entries.  The reference's head
(TenConvMlp with a 7x7 512->4096 conv, then timm's ClassifierHead, vgg_tt.py:52-88,137-141)
needs timm and is not part of the Tucker hot path; here the head is a global average pool and
one Linear(512, num_classes) named `head.fc`, and parity for this network is against the same
assembly in torch on the CPU.
"""
import torch
import torch.nn as nn

from . import ops
from ._lib import ERR_UNSUPPORTED, TdcError
from .resnet import Conv2dB200, _fold_bn, _tk_or_dense, round8
from .tkconv import TKConv2dC_B200

cfgs = {
    'vgg11': [64, 'M', 128, 'M', 256, 256, 'M', 512, 512, 'M', 512, 512, 'M'],
    'vgg13': [64, 64, 'M', 128, 128, 'M', 256, 256, 'M', 512, 512, 'M', 512, 512, 'M'],
    'vgg16': [64, 64, 'M', 128, 128, 'M', 256, 256, 256, 'M', 512, 512, 512, 'M', 512, 512, 512, 'M'],
    'vgg19': [64, 64, 'M', 128, 128, 'M', 256, 256, 256, 256, 'M', 512, 512, 512, 512, 'M', 512, 512, 512, 512, 'M'],
}


class HalfRanksVGG:
    """hp_dict with R1 = round8(0.5*in), R2 = round8(0.5*out) for every 3x3 conv except the first
    (3 input channels stay dense, as in inference/hp_dicts/tk_vgg16_bn_hp.py:3), in the key format
    of that file."""

    def __init__(self, cfg=cfgs['vgg16'], batch_norm=False, ratio=0.5):
        self.ranks = {}
        prev, idx = 3, 0
        for v in cfg:
            if v == 'M':
                idx += 1
                continue
            if prev != 3:
                self.ranks['features.%d.weight' % idx] = [round8(ratio * v), round8(ratio * prev)]
            idx += 3 if batch_norm else 2
            prev = v


class TKVGG(nn.Module):
    def __init__(self, cfg=cfgs['vgg16'], num_classes=1000, in_chans=3, batch_norm=False, hp_dict=None, precision="fp32"):
        super().__init__()
        hp_dict = hp_dict if hp_dict is not None else HalfRanksVGG(cfg, batch_norm)
        layers, prev, idx = [], in_chans, 0
        for v in cfg:
            if v == 'M':
                layers.append(nn.MaxPool2d(kernel_size=2, stride=2))
                idx += 1
                continue
            name = 'features.%d.weight' % idx
            if name in hp_dict.ranks:
                conv = TKConv2dC_B200(prev, v, kernel_size=3, padding=1, hp_dict=hp_dict, name=name)
            else:
                conv = Conv2dB200(prev, v, kernel_size=3, padding=1)
            layers += [conv, nn.BatchNorm2d(v), nn.ReLU(inplace=True)] if batch_norm else [conv, nn.ReLU(inplace=True)]
            idx += 3 if batch_norm else 2
            prev = v
        self.features = nn.Sequential(*layers)
        self.head = nn.Sequential()
        self.head.add_module("fc", nn.Linear(prev, num_classes))
        self.precision = precision
        for m in self.modules():            # the reference's _initialize_weights for conv / norm / linear
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')
                if m.bias is not None:
                    nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.constant_(m.bias, 0)

    def forward_features(self, x):
        if self.training:
            raise TdcError(ERR_UNSUPPORTED, "training mode is not built; call .eval()")
        if not x.is_cuda:
            raise TdcError(ERR_UNSUPPORTED, "TKVGG runs on CUDA tensors only")
        x = x.contiguous().float()
        mods = list(self.features)
        i = 0
        while i < len(mods):
            m = mods[i]
            if isinstance(m, nn.MaxPool2d):
                x = ops.pool2d(x, m.kernel_size, m.stride, m.padding)
                i += 1
                continue
            # conv [+ BatchNorm] + ReLU in the conv's own launch chain
            scale = shift = None
            j = i + 1
            if j < len(mods) and isinstance(mods[j], nn.BatchNorm2d):
                scale, shift = _fold_bn(mods[j])
                j += 1
            relu = j < len(mods) and isinstance(mods[j], nn.ReLU)
            x = _tk_or_dense(m, x, scale, shift, None, relu, self.precision)
            i = j + (1 if relu else 0)
        return x

    def forward(self, x):
        x = self.forward_features(x)
        return self.head.fc(torch.flatten(torch.nn.functional.adaptive_avg_pool2d(x, 1), 1))


def tkc_vgg16(hp_dict=None, num_classes=1000, batch_norm=False, precision="fp32"):
    """The feature stack of the reference's tkc_vgg16 / tkc_vgg16_bn (inference/vgg_tt.py:217-247)."""
    return TKVGG(cfgs['vgg16'], num_classes, 3, batch_norm, hp_dict, precision)
