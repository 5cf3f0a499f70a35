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


# The reference's six compiled operators have two bindings here (the compiled torch extension and
# ctypes, superl8_b200/_C.py); the GPU tests of these modules run once through each.
BOTH_BINDINGS = {"test_fwd_gpu", "test_decode_gpu", "test_bwd_gpu", "test_quant_gpu", "test_reference_cases_gpu"}


def pytest_generate_tests(metafunc):
    if metafunc.module.__name__ in BOTH_BINDINGS and "_sl8_binding" in metafunc.fixturenames:
        metafunc.parametrize("_sl8_binding", ["compiled", "ctypes"], indirect=True)


@pytest.fixture(autouse=True)
def _sl8_binding(request):
    name = getattr(request, "param", None)
    if name is None:
        yield
        return
    from superl8_b200 import _C
    if name == "compiled" and _C._ext is None:
        pytest.skip("the compiled extension is not built")
    prev = _C.use_binding(name)
    yield
    _C.use_binding(prev)


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
