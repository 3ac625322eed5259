"""croqtile_b200 — B200-native (sm_100a) GEMM family behind the Croqtile call signatures.

The compute lives in ``libcroq_b200.so`` (hand-written CUDA, C ABI declared in
``include/croq_b200.h``); this package is the thin host layer that binds it for
Python/torch callers. Import does not load the library; the first call does and
fails loudly if the library is missing.
"""
from . import _lib, schedule  # noqa: F401
from ._lib import CroqError  # noqa: F401
from .schedule import hilbert_schedule, row_major_schedule  # noqa: F401

__all__ = ["CroqError", "hilbert_schedule", "row_major_schedule", "schedule", "api"]


def __getattr__(name):
    if name == "api":
        import importlib
        return importlib.import_module(".api", __name__)
    raise AttributeError(name)
