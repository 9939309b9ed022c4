import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests refuse to run silently on a box without a device."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_sessionfinish(session, exitstatus):
    """With T3_PARITY_REPORT=<file>: the error measures every GPU parity check achieved, as JSON (the bars are asserted in
    the tests; this is the record of how far inside them the kernels are)."""
    path = os.environ.get("T3_PARITY_REPORT")
    if not path:
        return
    try:
        import json

        import gpu_util
        if gpu_util.ACHIEVED:
            with open(path, "w") as f:
                json.dump(gpu_util.ACHIEVED, f, indent=0)
    except Exception:
        pass
