"""TK-compressed ResNet on the B200 kernels — the assembly of the reference's TTResNet.

Mirrors inference/resnet_inet_tt.py: TTBasicBlock (:53-117), TTResNet (:287-394) and the
`tkc_resnet18` entry (:483-496) for the basic-block nets.  Module names, parameter names and
shapes are the reference's, so a state dict of `TTResNet(TTBasicBlock, [2,2,2,2],
conv=TKConv2dC, hp_dict=...)` loads with `load_state_dict` unchanged.  Which 3x3 convs are
Tucker convs is decided as there: the ones whose `layer{s}.{i}.conv{1,2}.weight` key is in
`hp_dict.ranks` (value `[R2, R1]`).

Every convolution runs on libtdc_b200.so: the Tucker convs as Tucker blocks, the stem (7x7,
stride 2) and the 1x1 stride-2 downsample convs through the same kernel family.  In eval mode
the BatchNorm that follows a conv is folded into that conv's last launch as a per-channel
scale and shift, together with the residual add and the ReLU (`forward` = one launch chain
per block, no elementwise passes); max-pool, global average pool and the classifier stay
torch ops.  Training-mode BatchNorm is not built: `forward` raises outside eval mode.
"""
import torch
import torch.nn as nn

from . import ops, tiles
from ._lib import ERR_UNSUPPORTED, W_CRSK, TdcError
from .dispatch import one_conv as _one_conv, tucker_strategy
from .tkconv import TKConv2dC_B200


def round8(v):
    return int(8 * round(v / 8.0))


class HalfRanks:
    """hp_dict with R1 = round8(0.5*in), R2 = round8(0.5*out) for every 3x3 conv of a basic-block
    ResNet — the benchmark's rank rule, in the format of inference/hp_dicts/tk_resnet18_hp.py:25-43."""

    def __init__(self, layers=(2, 2, 2, 2), ratio=0.5):
        self.ranks = {}
        inplanes = 64
        for s, (planes, n) in enumerate(zip((64, 128, 256, 512), layers), start=1):
            for i in range(n):
                cin = inplanes if i == 0 else planes
                self.ranks["layer%d.%d.conv1.weight" % (s, i)] = [round8(ratio * planes), round8(ratio * cin)]
                self.ranks["layer%d.%d.conv2.weight" % (s, i)] = [round8(ratio * planes), round8(ratio * planes)]
            inplanes = planes


class HalfRanksBottleneck:
    """hp_dict for a bottleneck ResNet: the 3x3 conv of every block (`layer{s}.{i}.conv2.weight`, width -> width)
    Tucker with R1 = R2 = round8(ratio*width); the 1x1 convs stay dense (inference/resnet_inet_tt.py:185-212 makes a
    conv Tucker only when its key is in `ranks`)."""

    def __init__(self, layers=(3, 4, 6, 3), ratio=0.5):
        self.ranks = {}
        for s, (planes, n) in enumerate(zip((64, 128, 256, 512), layers), start=1):
            for i in range(n):
                self.ranks["layer%d.%d.conv2.weight" % (s, i)] = [round8(ratio * planes), round8(ratio * planes)]


class Conv2dB200(nn.Conv2d):
    """nn.Conv2d parameters (`weight`, `bias`), forward on the B200 kernel."""

    def forward(self, x):
        return ops.conv2d(x, self.weight.detach(), None if self.bias is None else self.bias.detach(),
                          self.stride, self.padding)


def _fold_bn(bn):
    """Inference BatchNorm as y = x*scale + shift (fp64 arithmetic, rounded once); cached on the
    module until one of its tensors changes."""
    key = tuple((t._version, t.data_ptr()) for t in (bn.running_var, bn.running_mean, bn.weight, bn.bias)
                if t is not None)
    hit = getattr(bn, "_tdc_fold", None)
    if hit is not None and hit[0] == key:
        return hit[1], hit[2]
    scale, shift = _fold_bn_now(bn)
    bn._tdc_fold = (key, scale, shift)
    return scale, shift


def _fold_bn_now(bn):
    var, mean = bn.running_var.double(), bn.running_mean.double()
    g = bn.weight.double() if bn.weight is not None else torch.ones_like(var)
    b = bn.bias.double() if bn.bias is not None else torch.zeros_like(var)
    scale = g / torch.sqrt(var + bn.eps)
    return scale.float().contiguous(), (b - mean * scale).float().contiguous()


def _tk_or_dense(conv, x, scale, shift, residual, relu, precision="fp32"):
    """One conv module + folded BN (+ residual) (+ ReLU): a Tucker conv as its three launches with
    the epilogue on the last, a dense conv as one."""
    if conv.bias is not None:      # y = (conv + bias) * scale + shift  ->  conv * scale + (bias * scale + shift)
        b = conv.bias.detach() if scale is None else conv.bias.detach() * scale
        shift = b if shift is None else shift + b
    if isinstance(conv, TKConv2dC_B200):
        if tucker_strategy(conv, x, precision) == "dense":
            return _one_conv(conv, "dense", x, conv._dense_weight(), None, scale, shift, residual, relu, conv.stride[0], conv.padding[0], precision)
        z1 = _one_conv(conv, "first", x, conv.first_kernel, lambda: conv._factor_channel_last("first_kernel"), None, None, None, False, 1, 0, precision)
        z2 = _one_conv(conv, "core", z1, conv.core_kernel, conv._core_channel_last, None, None, None, False,
                       conv.stride[0], conv.padding[0], precision)
        return _one_conv(conv, "last", z2, conv.last_kernel, lambda: conv._factor_channel_last("last_kernel"), scale, shift, residual, relu, 1, 0, precision)
    return _one_conv(conv, "weight", x, conv.weight, None, scale, shift, residual, relu, conv.stride[0], conv.padding[0], precision)


class TKBasicBlock(nn.Module):
    """inference/resnet_inet_tt.py:53-117 (TTBasicBlock) with conv = TKConv2dC_B200."""
    expansion = 1

    def __init__(self, inplanes, planes, stride=1, downsample=None, stage=1, id=0, hp_dict=None):
        super().__init__()
        name = "layer%d.%d.conv1.weight" % (stage, id)
        if name in hp_dict.ranks:
            self.conv1 = TKConv2dC_B200(inplanes, planes, 3, stride=stride, padding=1, bias=False, hp_dict=hp_dict, name=name)
        else:
            self.conv1 = Conv2dB200(inplanes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.relu = nn.ReLU(inplace=True)
        name = "layer%d.%d.conv2.weight" % (stage, id)
        if name in hp_dict.ranks:
            self.conv2 = TKConv2dC_B200(planes, planes, 3, padding=1, bias=False, hp_dict=hp_dict, name=name)
        else:
            self.conv2 = Conv2dB200(planes, planes, 3, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.downsample = downsample
        self.stride = stride

    def forward(self, x):
        if self.training:
            raise TdcError(ERR_UNSUPPORTED, "training-mode BatchNorm is not built; call .eval()")
        s1, b1 = _fold_bn(self.bn1)
        s2, b2 = _fold_bn(self.bn2)
        prec = getattr(self, "precision", "fp32")
        out = _tk_or_dense(self.conv1, x, s1, b1, None, True, prec)
        identity = x
        if self.downsample is not None:
            sd, bd = _fold_bn(self.downsample[1])
            identity = _tk_or_dense(self.downsample[0], x, sd, bd, None, False, prec)
        return _tk_or_dense(self.conv2, out, s2, b2, identity, True, prec)


class TKBottleneck(nn.Module):
    """inference/resnet_inet_tt.py:155-237 (TTBottleneck, the v1.5 form: the stride sits on the 3x3 conv) with
    conv = TKConv2dC_B200 for the convs named in `hp_dict.ranks`, dense 1x1 / 3x3 otherwise."""
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, stage=1, id=0, hp_dict=None):
        super().__init__()
        width = planes

        def make(name, cin, cout, k, st):
            key = "layer%d.%d.%s.weight" % (stage, id, name)
            if key in hp_dict.ranks:
                return TKConv2dC_B200(cin, cout, k, stride=st, padding=k // 2, bias=False, hp_dict=hp_dict, name=key)
            return Conv2dB200(cin, cout, k, stride=st, padding=k // 2, bias=False)
        self.conv1 = make("conv1", inplanes, width, 1, 1)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = make("conv2", width, width, 3, stride)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = make("conv3", width, planes * self.expansion, 1, 1)
        self.bn3 = nn.BatchNorm2d(planes * self.expansion)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample
        self.stride = stride

    def forward(self, x):
        if self.training:
            raise TdcError(ERR_UNSUPPORTED, "training-mode BatchNorm is not built; call .eval()")
        prec = getattr(self, "precision", "fp32")
        s1, b1 = _fold_bn(self.bn1)
        s2, b2 = _fold_bn(self.bn2)
        s3, b3 = _fold_bn(self.bn3)
        out = _tk_or_dense(self.conv1, x, s1, b1, None, True, prec)
        out = _tk_or_dense(self.conv2, out, s2, b2, None, True, prec)
        identity = x
        if self.downsample is not None:
            sd, bd = _fold_bn(self.downsample[1])
            identity = _tk_or_dense(self.downsample[0], x, sd, bd, None, False, prec)
        return _tk_or_dense(self.conv3, out, s3, b3, identity, True, prec)


class TKResNet(nn.Module):
    """inference/resnet_inet_tt.py:287-394 (TTResNet) for basic blocks (`block=TKBasicBlock`) and bottleneck
    blocks (`block=TKBottleneck`)."""

    def __init__(self, layers=(2, 2, 2, 2), num_classes=1000, hp_dict=None, precision="fp32", block=None):
        super().__init__()
        block = block if block is not None else TKBasicBlock
        if hp_dict is None:
            hp_dict = HalfRanks(layers) if block is TKBasicBlock else HalfRanksBottleneck(layers)
        self.block = block
        self.inplanes = 64
        self.conv1 = Conv2dB200(3, 64, kernel_size=7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(kernel_size=3, stride=2, padding=1)
        self.layer1 = self._make_layer(64, layers[0], 1, 1, hp_dict)
        self.layer2 = self._make_layer(128, layers[1], 2, 2, hp_dict)
        self.layer3 = self._make_layer(256, layers[2], 2, 3, hp_dict)
        self.layer4 = self._make_layer(512, layers[3], 2, 4, hp_dict)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(512 * block.expansion, num_classes)
        for m in self.modules():        # the reference's init loop, resnet_inet_tt.py:335-340
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)
        self.set_precision(precision)

    def set_precision(self, precision):
        """"fp32" (default): every conv on the fp32 FMA kernels; "auto": large layers on tensor cores
        with split operands (fp32-level results), small ones on the fp32 kernels; "tf32x3" / "tf32":
        every stride-1 1x1 / 3x3 conv on tensor cores."""
        if precision not in ("fp32", "auto", "fp16x3", "tf32x3", "tf32"):
            raise ValueError("precision %r" % (precision,))
        self.precision = precision
        for m in self.modules():
            if isinstance(m, (TKBasicBlock, TKBottleneck)):
                m.precision = precision
        return self

    def _make_layer(self, planes, blocks, stride, stage, hp_dict):
        block, downsample = self.block, None
        if stride != 1 or self.inplanes != planes * block.expansion:
            downsample = nn.Sequential(Conv2dB200(self.inplanes, planes * block.expansion, 1, stride=stride, bias=False),
                                       nn.BatchNorm2d(planes * block.expansion))
        layers = [block(self.inplanes, planes, stride, downsample, stage=stage, id=0, hp_dict=hp_dict)]
        self.inplanes = planes * block.expansion
        for i in range(1, blocks):
            layers.append(block(self.inplanes, planes, stage=stage, id=i, hp_dict=hp_dict))
        return nn.Sequential(*layers)

    def forward(self, x):
        if self.training:
            raise TdcError(ERR_UNSUPPORTED, "training-mode BatchNorm is not built; call .eval()")
        if not x.is_cuda:
            raise TdcError(ERR_UNSUPPORTED, "TKResNet runs on CUDA tensors only")
        x = x.contiguous().float()
        s, b = _fold_bn(self.bn1)
        x = _tk_or_dense(self.conv1, x, s, b, None, True, self.precision)
        mp = self.maxpool      # nn.MaxPool2d kept as the module (state-dict and repr parity); computed by the pooling kernel
        x = ops.pool2d(x, mp.kernel_size, mp.stride, mp.padding)
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = torch.flatten(self.avgpool(x), 1)
        return self.fc(x)


def tkc_resnet18(hp_dict=None, num_classes=1000, precision="fp32"):
    """inference/resnet_inet_tt.py:483-496 without the checkpoint load."""
    return TKResNet((2, 2, 2, 2), num_classes, hp_dict, precision)


def tkc_resnet50(hp_dict=None, num_classes=1000, precision="fp32"):
    """inference/resnet_inet_tt.py:614-627 without the checkpoint load: bottleneck blocks [3, 4, 6, 3]; by default
    the 3x3 conv of every block is a Tucker conv with R = round8(0.5*width)."""
    return TKResNet((3, 4, 6, 3), num_classes, hp_dict, precision, block=TKBottleneck)


def fill_deterministic(module, seed=0, gain=1.0):
    """Every parameter and buffer from a generator seeded by (seed, its name): two models with
    the same state-dict keys — this one and the reference's — get identical values whatever their
    construction order.  Conv/Tucker kernels Kaiming-normal (fan_out) times `gain`, BatchNorm affine ~ (1, 0)
    +- 0.1, running mean ~ N(0, 0.1), running var in [0.5, 1.5], classifier ~ N(0, 0.01)."""
    import zlib
    sd = module.state_dict()
    for name in sorted(sd):
        t = sd[name]
        if not t.dtype.is_floating_point:
            continue
        g = torch.Generator().manual_seed((zlib.crc32(name.encode()) + seed) & 0x7FFFFFFF)
        if t.dim() == 4:
            fan_out = t.shape[0] * t.shape[2] * t.shape[3]
            v = torch.empty(t.shape).normal_(0.0, gain * (2.0 / fan_out) ** 0.5, generator=g)
        elif name.endswith("running_var"):
            v = torch.rand(t.shape, generator=g) + 0.5
        elif name.endswith("running_mean"):
            v = torch.randn(t.shape, generator=g) * 0.1
        elif name.endswith("weight") and t.dim() == 1:
            v = 1.0 + 0.1 * torch.randn(t.shape, generator=g)
        elif t.dim() == 2:
            v = torch.randn(t.shape, generator=g) * 0.01
        else:
            v = 0.1 * torch.randn(t.shape, generator=g)
        t.copy_(v.to(t.device))
    return module
