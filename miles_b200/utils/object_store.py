"""Object store for rollout -> trainer batches.

In the SPMD layout a rank trains on what it generated, so the default store is an in-process dict; a
file-backed store (shared filesystem, one ``.pt`` per key) serves disaggregated trainer / rollout ranks
and debugging.  Interface of the reference's miles/utils/object_store.py:99-165 (``put -> ref``,
``get(ref)``, ``delete``), with typed ragged-tensor encoding for the train-data dict.
"""
from __future__ import annotations

import itertools
import os
import uuid
from typing import Any, Optional

import torch

_RAGGED_INT = ("tokens", "loss_masks", "rollout_routed_experts", "rollout_indexer_topk")
_RAGGED_FLOAT = ("rollout_log_probs", "teacher_log_probs", "opd_reverse_kl", "values")


def encode_train_data(data: dict) -> dict:
    """Ragged python lists -> (flat tensor, offsets) pairs: compact and fast to (de)serialise."""
    out = {}
    for k, v in data.items():
        if k in _RAGGED_INT + _RAGGED_FLOAT and v is not None:
            dt = torch.int32 if k in _RAGGED_INT else torch.float32
            parts = [torch.as_tensor(x, dtype=dt).reshape(-1) for x in v]
            lens = torch.tensor([p.numel() for p in parts], dtype=torch.int64)
            out[k] = {"__ragged__": True, "flat": torch.cat(parts) if parts else torch.zeros(0, dtype=dt), "lens": lens,
                      "inner": [tuple(torch.as_tensor(x).shape[1:]) for x in v]}
        else:
            out[k] = v
    return out


def decode_train_data(enc: dict) -> dict:
    out = {}
    for k, v in enc.items():
        if isinstance(v, dict) and v.get("__ragged__"):
            parts = torch.split(v["flat"], v["lens"].tolist())
            out[k] = [p.reshape(-1, *inner) if inner else p for p, inner in zip(parts, v["inner"])]
        else:
            out[k] = v
    return out


class BaseObjectStore:
    def put(self, value: Any) -> str:
        raise NotImplementedError

    def get(self, ref: str) -> Any:
        raise NotImplementedError

    def delete(self, ref: str) -> None:
        raise NotImplementedError


class LocalObjectStore(BaseObjectStore):
    def __init__(self):
        self._d: dict = {}
        self._ids = itertools.count()

    def put(self, value: Any) -> str:
        ref = f"local-{next(self._ids)}"
        self._d[ref] = value
        return ref

    def get(self, ref: str) -> Any:
        return self._d[ref]

    def delete(self, ref: str) -> None:
        self._d.pop(ref, None)


class FileObjectStore(BaseObjectStore):
    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)

    def put(self, value: Any) -> str:
        ref = uuid.uuid4().hex
        tmp = os.path.join(self.root, ref + ".tmp")
        torch.save(encode_train_data(value) if isinstance(value, dict) else value, tmp)
        os.replace(tmp, os.path.join(self.root, ref + ".pt"))
        return ref

    def get(self, ref: str) -> Any:
        v = torch.load(os.path.join(self.root, ref + ".pt"), weights_only=False)
        return decode_train_data(v) if isinstance(v, dict) else v

    def delete(self, ref: str) -> None:
        try:
            os.remove(os.path.join(self.root, ref + ".pt"))
        except FileNotFoundError:
            pass


_INSTANCE: Optional[BaseObjectStore] = None


def init_instance(args=None) -> BaseObjectStore:
    global _INSTANCE
    backend = getattr(args, "object_store_backend", None) or "local"
    if backend in ("file", "mooncake") and getattr(args, "dump_details", None):
        _INSTANCE = FileObjectStore(os.path.join(args.dump_details, "object_store"))
    else:
        _INSTANCE = LocalObjectStore()
    return _INSTANCE


def get_instance() -> BaseObjectStore:
    global _INSTANCE
    if _INSTANCE is None:
        _INSTANCE = LocalObjectStore()
    return _INSTANCE
