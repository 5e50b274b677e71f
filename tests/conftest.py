import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def built_library():
    """The in-tree CUDA library, (re)built if its sources changed.  nvcc cross-compiles,
    so this also works on a machine without a GPU."""
    from landmark_b200.build import build_library

    return build_library()
