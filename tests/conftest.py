import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library; building it is part of the product build, not of the tests."""
    from nova_compiler_b200 import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def cuda():
    """torch with a usable CUDA device; GPU tests fail (not skip) when the library cannot run."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected but no CUDA device is visible"
    from nova_compiler_b200 import _lib
    _lib.check(_lib.load().nova_b200_init(0))
    return torch
