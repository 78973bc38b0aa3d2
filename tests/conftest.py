import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), '..'))
PKG = os.path.join(ROOT, 'flash-linear-attention_b200')
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200, sm_100a)')


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _no_bounded_wait_expired(request):
    """After every GPU test: none of the kernels' bounded waits gave up (a silent expiry would leave wrong results that a
    loose comparison might still accept).  The wait-expiry self-test clears the flag itself."""
    yield
    if 'gpu' not in request.keywords:
        return
    try:
        import torch
        if not torch.cuda.is_available():
            return
        import b200gdn
    except Exception:
        return
    b200gdn.device_status()
