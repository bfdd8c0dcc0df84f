import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.binding import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    from oracle.binding import Ref, ref_available
    if not ref_available():
        pytest.skip("oracle/_ref (the compiled reference) is not present")
    return Ref()


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library; built on demand when nvcc is available."""
    from vesper_b200 import capi
    if not os.path.exists(capi.LIB_PATH):
        from vesper_b200.build import build
        build()
    return capi.load()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for gpu-marked tests")
    return torch.device("cuda:0")
