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


class Ranks:
    """Stand-in for the hp_dict objects of inference/hp_dicts/*.py: `.ranks[name] -> [R2, R1]`."""

    def __init__(self, **ranks):
        self.ranks = dict(ranks)
