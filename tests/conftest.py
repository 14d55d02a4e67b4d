import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    """The CPU checker (oracle/counter_oracle.cpp).  Tests may use it; the product may not."""
    import oracle
    oracle.port.set_threads(len(os.sched_getaffinity(0)))
    return oracle.port


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def ctx():
    """A library context on cuda:0 sharing torch's current stream (GPU tests only)."""
    import torch
    from motifcl_b200 import Context
    assert torch.cuda.is_available(), "GPU test started without a CUDA device"
    torch.cuda.set_device(0)
    # a side stream made current for the whole session: torch's copies and the library's
    # kernels then share one in-order stream that can also be recorded into a batch
    side = torch.cuda.Stream(device=0)
    torch.cuda.set_stream(side)
    c = Context.on_torch_stream(0)
    yield c
    c.finish()
    c.close()
