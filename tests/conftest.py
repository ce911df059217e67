import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "ppopp23-tdc_b200"), os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


# the tensor-core launcher looks at its TDC_TC_* measurement switches only when this is set before its first launch
os.environ.setdefault("TDC_TC_TUNING", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built():
    """Builds (or finds) libtdc_b200.so and the C oracle once per session."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("tdc_build", os.path.join(ROOT, "ppopp23-tdc_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    mod.build_debug_bounds()
    import oracle
    oracle.build()
    return True
