import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ctx():
    import vulkanforge_b200 as vf
    c = vf.Context(0)
    yield c
    c.destroy()


@pytest.fixture(autouse=True)
def _poll_status(request):
    """After every GPU test the device status word must be clean (no clamped rows, no timeouts)."""
    yield
    if "gpu" in request.keywords and "ctx" in request.fixturenames:
        c = request.getfixturevalue("ctx")
        if not getattr(request.node, "expects_status", False):
            c.poll()
