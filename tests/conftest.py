"""Shared pytest configuration: the ``gpu`` marker and a few tiny helpers."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")
    config.addinivalue_line("markers", "distributed: spawns several ranks (gloo on CPU, NCCL on GPU)")
    config.addinivalue_line("markers", "slow: takes more than a few seconds")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from prism_infer_b200.ops import native

    if not native.available():
        pytest.fail("libprism_b200.so is missing on a GPU box: run python -m prism_infer_b200.ops.build")
    return torch.device("cuda:0")
