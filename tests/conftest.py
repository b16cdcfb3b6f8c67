import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(ROOT / "tests" / "golden" / "reference_vectors.pt", map_location="cpu")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built on demand; needs nvcc, not a GPU)."""
    from triton_kernels_b200 import _lib, build

    build.build()
    return _lib.load()
