"""flashrt_b200 — B200 (sm_100a) implementation of FlashRT's flow-matching / DiT denoise hot path.

Importing the package needs neither the CUDA library nor a GPU (the same lazy
convention as the reference's ``flash_rt/__init__.py:64-96``); the first kernel
call loads ``libflashrt_b200.so`` and raises if it has not been built.
"""
from __future__ import annotations

__version__ = "0.1.0"

_LAZY = {
    "load_model": ("flashrt_b200.api", "load_model"),
    "VLAModel": ("flashrt_b200.api", "VLAModel"),
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)
