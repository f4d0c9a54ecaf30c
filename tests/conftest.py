import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    # multi-process GPU tests first (they must run before this process owns a CUDA context), the allocation-free
    # entry-point test last
    def key(item):
        name = item.fspath.basename
        if name.startswith("test_zz"):
            return 2
        if "multigpu" in name:
            return 0
        return 1

    items.sort(key=key)
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if not has_gpu:
        skip = pytest.mark.skip(reason="no CUDA device")
        for item in items:
            if "gpu" in item.keywords:
                item.add_marker(skip)
