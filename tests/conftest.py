import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda_context():
    """One device context shared by the GPU tests of a session."""
    from webdnn_b200.backend import WebDNNCudaContext
    ctx = WebDNNCudaContext()
    ctx.initialize()
    yield ctx
    ctx.close()
