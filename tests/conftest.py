import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    """GPU tests fail (not skip) on a GPU box if CUDA is missing; on a CPU box they are deselected by -m."""
    return


@pytest.fixture(scope="session")
def cuda():
    import torch

    assert torch.cuda.is_available(), "this test needs a CUDA device"
    return torch.device("cuda:0")
