"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on CPU."""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc

    orc.lib()
    return orc


@pytest.fixture(scope="session")
def clib():
    """libcumpsgemm.so through ctypes (loads without a GPU)."""
    from cumpsgemm_b200 import _lib

    return _lib.load()


@pytest.fixture()
def handle():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cumpsgemm_b200 import api

    os.environ.pop("CUMPSGEMM_TILE_N", None)
    h = api.Handle()
    h.use_current_torch_stream()
    yield h
    status = h.kernel_status()
    h.destroy()
    assert status == 0, f"GEMM kernel reported bounded-wait status {status}"
