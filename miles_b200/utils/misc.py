"""Small shared helpers: dotted-path function loading, periodic-action predicate, singleton metaclass."""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
from typing import Any, Optional


def load_function(path: str) -> Any:
    """Resolve ``pkg.module.attr`` or ``/path/to/file.py:attr`` (or ``file.py::attr``) to an object.

    Same contract as the reference's ``load_function`` (miles/utils/misc.py:45-66): every pluggable hook
    (rollout fn, generate fn, reward fn, filters, loss, data source ...) is named by such a path.
    """
    if path is None:
        raise ValueError("function path is None")
    if ".py:" in path or path.endswith(".py"):
        file, _, attr = path.partition(":")
        attr = attr.lstrip(":")
        name = "_miles_user_" + os.path.splitext(os.path.basename(file))[0]
        spec = importlib.util.spec_from_file_location(name, file)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return getattr(mod, attr) if attr else mod
    module, _, attr = path.rpartition(".")
    if not module:
        raise ValueError(f"{path!r} is not a dotted path")
    return getattr(importlib.import_module(module), attr)


def should_run_periodic_action(rollout_id: int, interval: Optional[int], num_rollout_per_epoch: Optional[int] = None,
                               num_rollout: Optional[int] = None) -> bool:
    """True every ``interval`` rollouts, at an epoch boundary and at the very last rollout."""
    if interval is None:
        return False
    if num_rollout is not None and rollout_id == num_rollout - 1:
        return True
    step = rollout_id + 1
    if num_rollout_per_epoch is not None and step % num_rollout_per_epoch == 0:
        return True
    return step % interval == 0


class SingletonMeta(type):
    _instances: dict = {}

    def __call__(cls, *a, **k):
        if cls not in cls._instances:
            cls._instances[cls] = super().__call__(*a, **k)
        return cls._instances[cls]


def exec_command(cmd: str, capture: bool = False) -> Optional[str]:
    import subprocess

    r = subprocess.run(cmd, shell=True, check=True, capture_output=capture, text=True)
    return r.stdout if capture else None
