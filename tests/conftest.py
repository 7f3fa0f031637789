import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "needs_grad: the test differentiates through the layers")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle_lib():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def mn_lib():
    from minuet_b200 import build, _lib
    build.build()
    return _lib.load()


@pytest.fixture(autouse=True)
def _no_grad_unless_asked(request):
    """The parity tests are inference tests: they run without autograd, as the benchmark
    does.  Tests marked ``needs_grad`` differentiate through the layers."""
    import torch
    if "needs_grad" in request.keywords:
        yield
    else:
        with torch.no_grad():
            yield
