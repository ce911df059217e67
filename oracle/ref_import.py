"""Imports the reference's own inference/TKConv.py, unmodified, where the reference tree is
mounted (this development container only; the tree does not travel to a GPU box).

TKConv.py imports tensorly at module top (inference/TKConv.py:1-2,18) although TKConv2dC
touches it only when a dense weight is passed for decomposition.  tensorly is not installed
here, so two stub modules with the imported names are put in sys.modules first.  TEST
INFRASTRUCTURE ONLY: used by tests/golden/make_golden.py and by CPU tests that compare the
oracle with the reference module directly; skipped when the tree is absent.
"""
import os
import sys
import types

REFERENCE_ROOT = os.environ.get("TDC_REFERENCE_ROOT", "/root/reference")


def available():
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "inference", "TKConv.py"))


def _stub(name, **attrs):
    if name in sys.modules:
        return sys.modules[name]
    m = types.ModuleType(name)
    for k, v in attrs.items():
        setattr(m, k, v)
    sys.modules[name] = m
    return m


def _unavailable(*a, **k):
    raise RuntimeError("tensorly is not installed; only code paths that do not decompose dense weights work")


def import_tkconv():
    """Returns the reference's TKConv module (classes TKConv2dC, TKConv2dM, TKConv2dR)."""
    if not available():
        raise ImportError("reference tree not found at %s" % REFERENCE_ROOT)
    tl = _stub("tensorly", set_backend=lambda *_: None, tucker_to_tensor=_unavailable)
    dec = _stub("tensorly.decomposition", parafac=_unavailable, partial_tucker=_unavailable)
    tl.decomposition = dec
    inf = os.path.join(REFERENCE_ROOT, "inference")
    if inf not in sys.path:
        sys.path.insert(0, inf)
    import TKConv   # noqa: the reference's module name
    return TKConv


def import_resnet():
    """Returns the reference's resnet_inet_tt module (TTResNet, TTBasicBlock, ...), unmodified.
    Besides tensorly it imports timm only for its model registry decorator and for loading
    pre-trained checkpoints (inference/resnet_inet_tt.py:15-16,451-455); a stub with an identity
    `register_model` is enough to build and run the networks."""
    import_tkconv()
    reg = _stub("timm.models.registry", register_model=lambda f: f)
    models = _stub("timm.models", registry=reg)
    _stub("timm", models=models, create_model=_unavailable)
    import resnet_inet_tt   # noqa: the reference's module name
    return resnet_inet_tt


def import_svdconv():
    """Returns the reference's SVDConv module (SVDConv2dC, SVDConv2dM, SVDConv2dR); it needs torch and numpy only."""
    if not available():
        raise ImportError("reference tree not found at %s" % REFERENCE_ROOT)
    inf = os.path.join(REFERENCE_ROOT, "inference")
    if inf not in sys.path:
        sys.path.insert(0, inf)
    import SVDConv   # noqa: the reference's module name
    return SVDConv


def import_densenet():
    """Returns the reference's densenet_inet_tt module (TenDenseNet, ...), unmodified.  It takes four things from
    timm, which is not installed here (inference/densenet_inet_tt.py:5,14-18): the model registry decorator (an
    identity stub), `build_model_with_cfg` / `create_norm_act` / `BlurPool2d` (imported, never used by the default
    configuration: stubs that raise), and two building blocks that the default network does use and that are restated
    here from timm's documented behaviour — `BatchNormAct2d` = nn.BatchNorm2d followed by ReLU under BatchNorm2d's
    parameter names, and `create_classifier(num_features, num_classes, pool_type='avg')` = (global average pool +
    flatten, nn.Linear).  Everything else — the dense layers, blocks, transitions, the Tucker and SVD convs — is the
    reference's code."""
    import torch
    import torch.nn as nn
    import_tkconv()

    class BatchNormAct2d(nn.BatchNorm2d):
        def forward(self, x):
            return torch.relu(super().forward(x))

    class _GlobalAvgFlatten(nn.Module):
        def forward(self, x):
            return x.mean((2, 3))

    def create_classifier(num_features, num_classes, pool_type='avg'):
        assert pool_type == 'avg'
        return _GlobalAvgFlatten(), nn.Linear(num_features, num_classes)

    reg = _stub("timm.models.registry", register_model=lambda f: f)
    helpers = _stub("timm.models.helpers", build_model_with_cfg=_unavailable)
    layers = _stub("timm.models.layers", BatchNormAct2d=BatchNormAct2d, create_norm_act=_unavailable,
                   BlurPool2d=_unavailable, create_classifier=create_classifier)
    for name, val in (("BatchNormAct2d", BatchNormAct2d), ("create_norm_act", _unavailable), ("BlurPool2d", _unavailable),
                      ("create_classifier", create_classifier)):
        if not hasattr(layers, name):
            setattr(layers, name, val)
    models = _stub("timm.models", registry=reg)
    models.helpers, models.layers = helpers, layers
    data = _stub("timm.data", IMAGENET_DEFAULT_MEAN=(0.485, 0.456, 0.406), IMAGENET_DEFAULT_STD=(0.229, 0.224, 0.225))
    timm = _stub("timm", models=models, create_model=_unavailable)
    timm.data = data
    import densenet_inet_tt   # noqa: the reference's module name
    return densenet_inet_tt


def import_hp_dict(module_name):
    """A module of the reference's inference/hp_dicts (e.g. "tk_densenet121_hp"): plain Python dictionaries."""
    import importlib.util
    path = os.path.join(REFERENCE_ROOT, "inference", "hp_dicts", module_name + ".py")
    spec = importlib.util.spec_from_file_location("tdc_ref_" + module_name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class Ranks:
    """Stand-in for the hp_dict objects of inference/hp_dicts/*.py: `.ranks[name] -> [R2, R1]`."""

    def __init__(self, **ranks):
        self.ranks = dict(ranks)
