"""Loader of ``miles_b200._native`` (host-only C++ runtime: scheduler / page pool, quorum store, router table).

The module has no CUDA or PyTorch dependency; it is compiled in-tree on first use if the shared object is missing
or older than its sources."""
from __future__ import annotations

import importlib

_mod = None


def load():
    global _mod
    if _mod is None:
        from .. import _build

        if _build.native_needs_build():
            _build.build_native()
        _mod = importlib.import_module("miles_b200._native")
    return _mod
