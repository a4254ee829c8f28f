import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "plain")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    """Tests marked gpu fail loudly without a device rather than pass on a fallback;
    when no device exists and -m gpu was not asked for, they are deselected by -m "not gpu"."""
    return


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    assert torch.cuda.is_available(), "this test needs a CUDA device"
    from binfer_b200.csrc import ops
    ops.lib()
    return torch.device("cuda:0")
