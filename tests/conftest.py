import os
import sys

import pytest

# The reference's batch-parallel GEMM deadlocks unless its OpenMP team divides the batch (batch >= 4), and its
# scratch tables hold 32 threads: the live-reference checks use batches of 1 to 4, so pin the team to 4 before any
# OpenMP runtime starts.
os.environ["OMP_NUM_THREADS"] = "4"

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()
