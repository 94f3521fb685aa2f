import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def backend():
    """The engine on cuda:0 through the C ABI. Fails (never skips) when it cannot be opened."""
    import oxinfer_b200 as ob

    be = ob.Backend(0)
    yield be
    be.close()
