"""Shared fixtures. Tests marked `gpu` need a B200 and the built libmfx.so; everything else runs on CPU."""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a) and the built libmfx.so")


@pytest.fixture(scope="session")
def lib_built():
    """Build libmfx.so if it is missing (nvcc cross-compiles without a GPU)."""
    from mflux_b200 import build

    return build.build()


def seeded(seed: int):
    import torch

    return torch.Generator(device="cpu").manual_seed(seed)
