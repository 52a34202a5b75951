import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libhyacin_ref.so")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def hy():
    """Handle on the product library (libhyacin.so); no fallback if it is missing."""
    import torch
    from hyacinth_b200 import api
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    h = api.Hyacin(stream=0)
    yield h
    h.destroy()


@pytest.fixture(scope="session")
def ref():
    """Handle on the reference's own CUDA library when it was built into oracle/_ref (checker only)."""
    import torch
    from hyacinth_b200 import api
    if not os.path.exists(REF_LIB):
        pytest.skip("reference library not built (oracle/_ref/libhyacin_ref.so)")
    assert torch.cuda.is_available()
    h = api.Hyacin(lib_path=REF_LIB, stream=0)
    yield h
    h.destroy()
