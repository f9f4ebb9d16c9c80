import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def reference_kernels(monkeypatch):
    """Put the plain references of `tests/kernel_refs.py` in the kernels' place and lift the CUDA-only
    check, so that the step function, the cache and the loops above them can run on the CPU. The package
    itself has no such path."""
    from qwenforge_b200 import ops
    from qwenforge_b200.engine import model as model_module
    from tests import kernel_refs

    for name, fn in kernel_refs.ALL.items():
        monkeypatch.setattr(ops, name, fn)
    monkeypatch.setattr(ops, "require_cuda", lambda device, what="": None)
    monkeypatch.setattr(model_module, "prepare", lambda names: None)
    yield
