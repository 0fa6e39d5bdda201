import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def restatement():
    from oracle import oracle as O
    return O.restatement()


@pytest.fixture(scope="session")
def checker():
    """The compiled reference when its binary is present, else the plain-C restatement."""
    from oracle import oracle as O
    return O.best_checker()


@pytest.fixture(scope="session")
def gpu_ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from edge0_b200 import moe
    ctx = moe.Context(0)
    yield ctx
    ctx.close()
