import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")


@pytest.fixture(scope="session")
def native_lib():
    """The C-ABI library, built in-tree if missing (nvcc cross-compiles without a GPU)."""
    from kernelcodegen_b200 import build, capi

    build.build()
    return capi.load()


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "kat_small.npz")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("test marked gpu but no CUDA device is visible")
    from kernelcodegen_b200 import build

    build.build()
    return torch.device("cuda:0")
