import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from pj_testlib import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def native():
    """The built product library (compiled on demand; nvcc cross-compiles without a GPU)."""
    from pj_testlib import build, pj

    build.build_library()
    build.build_generator()
    return pj


@pytest.fixture(scope="session")
def ctx(native):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    c = native.Context(device=0)
    yield c
    c.close()
