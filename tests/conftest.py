"""Shared pytest configuration: the `gpu` marker and a few helpers."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) and the built libcroq_b200.so")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.lib()
    return o


@pytest.fixture(scope="session")
def golden():
    return {p.stem: np.load(p) for p in GOLDEN.glob("*.npz")}


@pytest.fixture(scope="session")
def croq():
    """The built library; GPU tests fail (not skip) when it is missing."""
    from croqtile_b200 import _lib
    return _lib.load()
