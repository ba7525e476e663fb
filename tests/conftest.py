import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session", autouse=True)
def no_kernel_wait_ran_out():
    """After the whole session: no kernel of the library gave up on one of its bounded waits (such
    a launch would have produced undefined output without any other sign)."""
    yield
    import torch
    if torch.cuda.is_available():
        from deepshift_b200 import _ffi, kernels
        if _ffi._lib is not None:
            assert kernels.last_kernel_error() == 0
