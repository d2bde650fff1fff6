"""Test configuration: the ``gpu`` marker and a helper to skip without a B200."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """``BUX_SHARD=i/n`` keeps the tests whose id hashes to shard i of n, so that n runners split
    the suite between them (every test lands in exactly one shard)."""
    shard = os.environ.get("BUX_SHARD")
    if not shard:
        return
    import zlib

    i, n = (int(x) for x in shard.split("/"))
    keep = [item for item in items if zlib.crc32(item.nodeid.encode()) % n == i]
    config.hook.pytest_deselected(items=[item for item in items if item not in keep])
    items[:] = keep


@pytest.fixture
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _kernel_checks(request):
    """With BUX_KERNEL_CHECKS=1 every kernel output sits between guard regions; they are
    verified after each GPU test."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    from bux_b200.ops import checks

    if checks.enabled():
        import torch

        if torch.cuda.is_available():
            torch.cuda.synchronize()
        checks.verify()
