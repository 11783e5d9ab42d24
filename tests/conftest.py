import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# device-side time-outs and span-id range errors surface as exceptions right after each call
os.environ.setdefault("KD_CHECK_STATUS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA sm_100 device (run on the GPU box)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library is built once per session (nvcc cross-compiles without a GPU)."""
    from kerneldev_b200.build import build
    build()
