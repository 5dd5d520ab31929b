import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, 'tests', 'golden')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200); run with -m gpu')


@pytest.fixture(scope='session')
def golden_dir():
    return GOLDEN


@pytest.fixture(autouse=True)
def _no_device_timeouts(request):
    """After every GPU test: fail if a kernel reported that one of its bounded waits expired."""
    yield
    if request.node.get_closest_marker('gpu') is not None:
        import torch
        if torch.cuda.is_available():
            import hyperattention_b200 as ha
            ha.check_device_status()
