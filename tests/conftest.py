import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on the B200 box)")


@pytest.fixture(autouse=True)
def _reset_globals():
    from chatlearn_b200.utils import global_vars
    global_vars.reset()
    yield
    global_vars.reset()
