import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qwenny_b200.ops import Context
    c = Context(0)
    yield c
    torch.cuda.synchronize()
    assert c.device_error() == 0, "a kernel gave up a bounded wait"


@pytest.fixture(scope="session")
def ref():
    """The reference's own kernels (oracle/_ref), loaded on the GPU."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import ref_cuda
    if not ref_cuda.available():
        pytest.skip("oracle/_ref not built (python oracle/build_ref.py)")
    return ref_cuda.RefModule()
