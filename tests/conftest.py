"""Test configuration: markers, library build, backend helpers.

``-m "not gpu"`` runs everything that needs no GPU (the daemon, the engine and
the runtime are exercised through the host backend: CPU threads stand in for
thread blocks and POSIX shared memory for peer memory).  ``-m gpu`` runs on a
B200 and must load ``dfccl_b200/lib/libdfccl.so``.
"""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
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
    for it in items:
        if "gpu" in it.keywords and n == 0:
            it.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in it.keywords and n < 2:
            it.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(scope="session")
def native():
    from dfccl_b200 import native as nv
    nv.lib()
    return nv


@pytest.fixture()
def host_backend(native):
    native.set_backend("host")
    yield native
    native.set_backend("cuda" if _cuda_count() else "host")
