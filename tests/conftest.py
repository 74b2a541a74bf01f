import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped where no CUDA device exists (the CPU-only check box)."""
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a
    temporary folder: {name: (dir, config dict)}."""
    from tiny_configs import TINY, write_tiny
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name in TINY:
        out[name] = (write_tiny(name, str(root / name)), TINY[name]["config"])
    return out
