import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on a B200 with `-m gpu`)')


@pytest.fixture(scope='session')
def c_oracle():
    """The compiled C oracle (built on demand with gcc)."""
    from oracle import c_oracle as co
    co.build()
    return co


@pytest.fixture(scope='session')
def bsx():
    """The C-ABI library, built on demand (nvcc cross-compiles without a GPU)."""
    from brainstate_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from brainstate_b200.build import build_library
        build_library()
    return _lib.lib()


@pytest.fixture(scope='session')
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail('a test marked gpu ran without a CUDA device')
    return torch.device('cuda:0')
