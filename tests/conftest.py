"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA library through its
C ABI; everything else runs on CPU (oracle vs golden vectors, host logic, exported symbols)."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        have_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def built_library():
    """Build (if stale) and load the shared library."""
    from helion_b200 import _lib, build

    build.build()
    return _lib.load()


def load_golden(name: str):
    return np.load(GOLDEN / f"{name}.npz")


GEMM_GOLDEN = [
    "gemm_256_colmajor",
    "gemm_256_rowmajor",
    "gemm_ragged_colmajor",
    "gemm_ragged_rowmajor",
    "gemm_skinny_colmajor",
]
ATTN_GOLDEN = ["attn_b1h2s128d64", "attn_b2h4s256d64", "attn_b1h2s512d128", "attn_b1h1s80d64"]
