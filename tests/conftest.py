import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (ROOT / "pytorch-apple_b200", ROOT, ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def fake_native():
    """Route the runtime to the host stand-in library (CPU tests of the host logic)."""
    from cuda_runtime import native
    from fake_b200nn import FakeLibrary

    lib = FakeLibrary()
    native.install_test_library(lib, "cpu")
    yield lib
    native.install_test_library(None)


@pytest.fixture(scope="session")
def native_lib():
    """The real library, built on demand (nvcc cross-compiles without a GPU)."""
    from cuda_runtime import native

    if not native.library_path().exists():
        import build_native

        build_native.build()
    return native.load()
