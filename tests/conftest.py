import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def cuda_lib():
    """Build (if stale) and load the CUDA library; a missing library is a hard failure."""
    from radiance_meshes_b200.csrc import build
    build.build()
    from radiance_meshes_b200 import _lib
    return _lib.load()
