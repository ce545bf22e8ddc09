import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def ctx():
    """One library context on cuda:0 for the GPU tests; fails loudly without the CUDA extension."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import tensor_adapt_b200 as ta
    c = ta.Context(0)
    yield c
    torch.cuda.synchronize()
    c.check_device()
    c.close()
