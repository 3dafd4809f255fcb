import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def built_lib():
    """libqeng.so, built in-tree if it is missing or stale (nvcc cross-compiles without a GPU)."""
    from cyb_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def oracle_c():
    from oracle import cport
    cport.build()
    return cport


@pytest.fixture(scope="session")
def ctx(built_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cyb_b200 import qeng
    c = qeng.Context(0)
    yield c
    c.device_status()
    c.close()
