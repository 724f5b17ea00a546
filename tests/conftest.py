"""pytest configuration: registers the ``gpu`` marker and makes the package importable in-tree."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE_DIR = os.path.join(ROOT, "kohakufa-cute_b200")
for path in (ROOT, PACKAGE_DIR):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (sm_100a) and the built CUDA library")


def pytest_collection_modifyitems(config, items):
    import torch

    if config.pluginmanager.hasplugin("timeout"):
        # a test that stops making progress ends with a stack dump instead of holding the GPU
        for item in items:
            if item.get_closest_marker("timeout") is None:
                item.add_marker(pytest.mark.timeout(600))
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
