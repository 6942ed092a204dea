import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # the file holding the no-allocation entry point's test must run last
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if torch.cuda.get_device_capability(0)[0] != 10:
        pytest.skip("needs sm_100 (B200)")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def oracle():
    from oracle import fp4_oracle as O

    O.build()
    return O
