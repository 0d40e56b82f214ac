import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def _cuda_count() -> int:
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_collection_modifyitems(config, items):
    n = _cuda_count()
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(scope="session", autouse=True)
def _native_lib():
    """Build the native library once per session if it is missing (nvcc cross-compiles without a GPU)."""
    from hccl_b200 import _lib

    if not _lib.LIB_PATH.exists():
        from hccl_b200.utils import build

        build.build_native()
    os.environ.setdefault("HCCL_DEVICE_WAIT_TIMEOUT_MS", "20000")
    return _lib.lib()
