import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for sub in ("deep-learning_b200", "oracle", "tests"):
    p = os.path.join(ROOT, sub)
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def gpu_ctx():
    """One CUDA context for the whole GPU session.  Creation fails loudly when
    the library is not built or no sm_100 device is present."""
    import dlb200

    ctx = dlb200.Context(0)
    yield ctx
    ctx.sync()
