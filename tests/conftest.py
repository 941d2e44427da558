"""Test configuration: the ``gpu`` marker, device parametrisation and seeding."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: test needs a CUDA device (B200)')


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


# Every op test runs its body on the CPU (plain PyTorch path) and, on a GPU box,
# on CUDA (native kernels) against the same inline oracle.
DEVICES = [pytest.param('cpu', id='cpu'), pytest.param('cuda', id='cuda', marks=pytest.mark.gpu)]


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(1234)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(1234)
    yield
    if torch.cuda.is_available():
        from megablocks_b200.utils import status
        status.check()   # no kernel may have abandoned a wait
    from megablocks_b200.layers import moe, router
    moe.clear_load_balancing_loss()
    router.clear_router_zloss()
