import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def gpu_lib():
    """The built library with the B200 backend active; fails loudly otherwise."""
    import eshkol_b200 as eb
    lib = eb.load_library()
    assert lib.eshkol_gpu_init() == 1, "eshkol_gpu_init did not find a usable sm_100 device"
    return lib
