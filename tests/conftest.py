import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def native_lib():
    """The built C-ABI library (built on demand; nvcc cross-compiles without a GPU)."""
    from torch_mlu_b200 import _cabi, build
    if not os.path.exists(_cabi.LIB_PATH):
        build.build_native()
    return _cabi.load()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    assert torch.cuda.get_device_capability(0)[0] == 10, "these kernels are built for sm_100a only"
    return torch.device("cuda", 0)
