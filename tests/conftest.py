import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    # CPU engines of the tests compare token sequences of tiny random models, whose top logits
    # lie close together. With several intra-op threads the math library splits a reduction
    # according to the load of the machine, the sums round differently from run to run and a
    # near-tie flips; one thread makes every CPU matmul reproducible.
    try:
        import torch
        torch.set_num_threads(1)
    except Exception:
        pass


def pytest_collection_modifyitems(config, items):
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
