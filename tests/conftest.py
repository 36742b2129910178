import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def plugin():
    """The CUDA plugin, loaded through its C ABI.  No fallback: a missing
    library or a missing GPU fails the test."""
    import mlx_b200
    return mlx_b200.Plugin(require_gpu=True)


@pytest.fixture()
def ctx(plugin):
    c = plugin.context(0)
    yield c
    c.close()
