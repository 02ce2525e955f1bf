"""In-process hand-off of weight buckets between a trainer and an engine HTTP front that live in the same
process (the analogue of serialised CUDA-IPC handles in the reference's colocate mode,
miles/backends/megatron_utils/update_weight/update_weight_from_tensor.py:450-545)."""
from __future__ import annotations

import itertools
import threading

_LOCK = threading.Lock()
_BUCKETS: dict = {}
_IDS = itertools.count()


def put_bucket(named_tensors) -> int:
    with _LOCK:
        i = next(_IDS)
        _BUCKETS[i] = list(named_tensors)
        return i


def take_bucket(bucket_id: int):
    with _LOCK:
        return _BUCKETS.pop(int(bucket_id))
