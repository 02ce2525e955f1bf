"""Loader of the in-tree sm_100a extension ``miles_b200/_C.so``.

The extension is mandatory on a machine with a GPU: if it is missing it is built once with nvcc, and if
that fails the import raises instead of silently falling back to eager PyTorch.  On a CPU-only machine
``load()`` returns ``None`` and the pure-PyTorch reference implementations in ``ops.reference`` are used
(this is what the CPU/gloo tests exercise).
"""
from __future__ import annotations

import importlib.util
import os
import threading
from pathlib import Path

_LOCK = threading.Lock()
_MOD = None
_TRIED = False


def _import_so(path: Path):
    import torch  # noqa: F401  (libtorch symbols must be loaded first)

    spec = importlib.util.spec_from_file_location("miles_b200._C", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load(required: bool | None = None):
    """Return the extension module, or ``None`` when no GPU is present and it is not required."""
    global _MOD, _TRIED
    if _MOD is not None:
        return _MOD
    with _LOCK:
        if _MOD is not None:
            return _MOD
        import torch

        has_gpu = torch.cuda.is_available()
        if required is None:
            required = has_gpu
        if not required and not has_gpu and os.environ.get("MILES_B200_LOAD_EXT", "0") != "1":
            return None
        from .. import _build

        if _build.needs_build():
            if _TRIED:
                raise RuntimeError("miles_b200._C could not be built earlier in this process")
            _TRIED = True
            _build.build(verbose=True)
        _MOD = _import_so(_build.TARGET)
        return _MOD


def available() -> bool:
    import torch

    return torch.cuda.is_available() and load() is not None
