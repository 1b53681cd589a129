import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(autouse=True)
def _kernel_status_clean(request):
    """After every GPU test, no kernel may have recorded an error (bounded wait ran out, bad argument)."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from llmc_b200 import _lib
    status = _lib.read_status(clear=True)
    assert status == 0, "a kernel recorded error status 0x%08x" % status
