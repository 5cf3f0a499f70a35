import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


@pytest.fixture(scope="session")
def device():
    assert torch.cuda.is_available()
    return torch.device("cuda", 0)


def from_bits(arr, dtype_name):
    """Inverse of the golden files' raw-bit storage of 16-bit floats."""
    t = torch.from_numpy(arr.copy())
    if dtype_name == "float16":
        return t.view(torch.float16)
    if dtype_name == "bfloat16":
        return t.view(torch.bfloat16)
    return t
