import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box only)")


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library, built in-tree if stale (nvcc cross-compiles without a GPU)."""
    from metalaudio_b200 import _lib, build
    build.build_library()
    return _lib.load()


@pytest.fixture(scope="session")
def device(lib):
    """One AudioDevice (CUDA context) shared by the GPU tests."""
    from metalaudio_b200 import AudioDevice
    dev = AudioDevice()
    yield dev
    dev.close()
