import importlib
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
importlib.import_module("amdgpu-arch-gemm_b200")  # puts generator/, runner/, tuner/ on sys.path

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def built():
    """Runner library + kernels: built once per session if the in-tree artefacts are missing."""
    from runner import api
    import kernels

    api.build_library()
    return kernels


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
