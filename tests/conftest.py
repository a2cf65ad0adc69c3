import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc

    orc.build()
    return orc


@pytest.fixture(scope="session")
def plugin_path():
    """The delegate plugin, built on first use (skips where neither the library nor the headers exist)."""
    from litert_b200 import build_delegate

    p = build_delegate.build()
    if p is None:
        pytest.skip("delegate library not built and LiteRT headers absent")
    return p
