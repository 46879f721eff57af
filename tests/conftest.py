"""Shared pytest configuration: the `gpu` marker and a few fixtures."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the native kernel library")
    config.addinivalue_line("markers", "multi_gpu: needs two or more CUDA devices")
    config.addinivalue_line("markers", "slow: long-running test")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multi_gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def seed():
    torch.manual_seed(0)
    return 0
