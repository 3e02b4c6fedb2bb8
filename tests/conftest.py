import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def kat():
    with open(os.path.join(ROOT, "tests", "golden", "reference_kat.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    return O


@pytest.fixture(scope="session")
def device():
    """The CUDA device under test. Fails (does not skip) when the library or the GPU is missing: a GPU test
    that silently passes without running the CUDA path would prove nothing."""
    from neureka_b200.device import CudaDevice
    assert CudaDevice.count() > 0, "no CUDA device visible"
    return CudaDevice.get(0)
