"""Test configuration.  ``gpu`` marks tests that need at least one CUDA device (B200)."""

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("OMP_NUM_THREADS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch

    have = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for item in items:
        if item.get_closest_marker("multigpu") and have < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 GPUs"))
