import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def finish_rank(dist) -> None:
    """End of a gloo / NCCL worker's ``finally`` block. The closing barrier runs only when the body succeeded: a rank
    that raised leaves with its traceback instead of parking in a barrier (or making its peers wait for one), so a
    broken test fails at the parent's first poll with the cause on stderr, not at a timeout."""
    import sys

    if sys.exc_info()[0] is None:
        dist.barrier()
    dist.destroy_process_group()
