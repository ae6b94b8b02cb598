import importlib
import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (REPO, os.path.join(REPO, "oracle"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def hkv():
    """The host package (its directory name is not a Python identifier)."""
    return importlib.import_module("hector-engine_b200")


@pytest.fixture(scope="session")
def oracle():
    import hkv_oracle
    hkv_oracle.load()
    return hkv_oracle


@pytest.fixture(scope="session")
def cuda(hkv):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    hkv._capi.load()  # the native library must be the thing under test
    torch.cuda.set_device(0)
    return torch
