import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device; run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on demand."""
    from oracle import build_oracle
    build_oracle.build_oracle()
    from oracle import oracle as O
    return O


@pytest.fixture(scope="session")
def native_lib():
    """The CUDA library, built on demand (nvcc cross-compiles without a GPU)."""
    from blaze_b200 import build
    build.build()
    from blaze_b200 import _native
    return _native.lib()


@pytest.fixture(scope="session")
def cuda_device(native_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    if torch.cuda.get_device_capability(0)[0] != 10:
        pytest.fail("GPU tests need an sm_100 device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
