"""pytest configuration: the `gpu` marker (tests that need a B200) and the repository root on sys.path."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (sm_100a); run with -m gpu on a B200 box")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, where no GPU is visible (the CPU container)."""
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
