import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")


@pytest.fixture(scope="session")
def built_lib():
    """Path of the in-tree shared library, (re)built if sources are newer."""
    from megaqwen_b200.csrc.build import build
    return build()
