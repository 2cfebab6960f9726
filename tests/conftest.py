import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def built_artifacts():
    """Build what is missing (nvcc and gcc work without a GPU); prebuilt files are used as they are."""
    from cudadma_b200 import build
    need = [os.path.join(ROOT, "cudadma_b200", "libcudadma_b200.so"),
            os.path.join(ROOT, "tests", "csrc", "libcudadma_apitest.so"),
            os.path.join(ROOT, "tests", "csrc", "libcudadma_checked_probe.so"),
            os.path.join(ROOT, "oracle", "liboracle.so")]
    if not all(os.path.exists(p) for p in need):
        if shutil.which("nvcc") or os.path.exists(build.NVCC):
            build.build_all(reference=False)
    return need
