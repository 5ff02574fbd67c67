import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def backend():
    """The CUDA backend on cuda:0.  GPU tests fail (not skip) if the library is missing."""
    import torch
    from torch_engine_b200 import ops
    assert torch.cuda.is_available(), "GPU test run without a GPU"
    be = ops.Backend(0, workspace_bytes=5 << 30)   # 16384^3 in 3xTF32 mode packs 4 GiB of planes
    yield be
    be.check_device_status()
    be.close()
