"""Weight update over a dedicated process group: the trainer broadcasts, engines in other processes receive.

This is the transport for *disaggregated* rollout engines (their own processes / GPUs, reachable over HTTP): the
trainer's source rank and every engine rank join a process group that exists only for weight updates
(``init_update_group``; NCCL between GPUs, gloo on CPU), independent of either side's default group. One update:

    pause_generation -> flush_cache -> for each bucket (<= buffer bytes):
        POST /update_weights_from_distributed {names, dtypes, shapes, group_name}     (engine starts receiving)
        broadcast(tensor, src=0) for every tensor of the bucket                        (trainer sends)
    -> update_weight_version -> continue_generation

Dense parameters go first, expert parameters second; under expert parallelism the source rank first gathers the
experts of a bucket over the EP group so that engines see whole tensors.

Reference counterpart: miles/backends/megatron_utils/update_weight/update_weight_from_distributed/broadcast.py:21-291
and mixin.py:98-226 (group bring-up), miles/utils/distributed_utils.py:40-93 (the stand-alone group helper).
"""
from __future__ import annotations

import datetime
from typing import Iterable, Optional, Sequence

import torch
import torch.distributed as dist

from ..models.hf_mapping import param_or_hf_view

_GROUPS: dict = {}


def init_update_group(master_address: str, master_port: int, rank: int, world_size: int, group_name: str,
                      backend: str = "nccl", timeout_s: float = 300.0):
    """A process group outside the default world: rendezvous on its own TCP store, ranks 0..world_size-1."""
    from torch.distributed.distributed_c10d import PrefixStore, _new_process_group_helper, _world, rendezvous

    timeout = datetime.timedelta(seconds=timeout_s)
    it = rendezvous(f"tcp://{master_address}:{master_port}", rank, world_size, timeout=timeout)
    store, rank, world_size = next(it)
    store.set_timeout(timeout)
    store = PrefixStore(group_name, store)
    kw = dict(group_name=group_name, timeout=timeout)
    try:
        pg, _ = _new_process_group_helper(world_size, rank, [], backend, store, backend_options=None, **kw)
    except TypeError:  # older argument name
        pg, _ = _new_process_group_helper(world_size, rank, [], backend, store, pg_options=None, **kw)
    _world.pg_group_ranks[pg] = {i: i for i in range(world_size)}
    _GROUPS[group_name] = pg
    return pg


def get_update_group(group_name: str):
    return _GROUPS[group_name]


def destroy_update_group(group_name: str) -> bool:
    pg = _GROUPS.pop(group_name, None)
    if pg is None:
        return False
    try:
        dist.destroy_process_group(pg)
    except Exception:
        pass
    return True


_DT = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "uint8": torch.uint8,
       "int32": torch.int32, "float8_e4m3fn": torch.float8_e4m3fn}


def dtype_name(dt: torch.dtype) -> str:
    return str(dt).replace("torch.", "")


def iter_buckets(named: Iterable, max_bytes: int):
    """Group (name, tensor) pairs into buckets of at most ``max_bytes`` (a single larger tensor is its own bucket)."""
    cur, size = [], 0
    for name, t in named:
        nb = t.numel() * t.element_size()
        if cur and size + nb > max_bytes:
            yield cur
            cur, size = [], 0
        cur.append((name, t))
        size += nb
    if cur:
        yield cur


def bucket_header(bucket: Sequence, group_name: str, weight_version: Optional[int] = None) -> dict:
    return {"names": [n for n, _ in bucket], "dtypes": [dtype_name(t.dtype) for _, t in bucket],
            "shapes": [list(t.shape) for _, t in bucket], "group_name": group_name, "weight_version": weight_version}


def send_bucket(bucket: Sequence, group_name: str) -> int:
    pg = _GROUPS[group_name]
    works = [dist.broadcast(t.contiguous(), src=0, group=pg, async_op=True) for _, t in bucket]
    for w in works:
        w.wait()
    return sum(t.numel() * t.element_size() for _, t in bucket)


@torch.no_grad()
def receive_bucket(header: dict, store, device=None) -> int:
    """Engine side of one bucket: receive every tensor and copy it into the parameter of the same name."""
    pg = _GROUPS[header["group_name"]]
    dev = device or store.device
    n = 0
    for name, dt, shape in zip(header["names"], header["dtypes"], header["shapes"]):
        buf = torch.empty(shape, dtype=_DT[dt], device=dev)
        dist.broadcast(buf, src=0, group=pg)
        dst = param_or_hf_view(store.global_cfg, store, name)  # native or HuggingFace tensor name
        if tuple(dst.shape) != tuple(buf.shape):
            raise ValueError(f"{name}: received shape {tuple(buf.shape)} but the engine holds {tuple(dst.shape)}")
        dst.copy_(buf.to(dst.dtype))
        n += 1
    return n


class BroadcastWeightUpdater:
    """Trainer side. ``engines`` are clients with ``post(path, json) -> dict`` (blocking) and
    ``post_async(path, json) -> handle`` whose ``result()`` waits; ``engine_world_sizes[i]`` ranks per engine."""

    def __init__(self, actor, engines: Sequence, group_name: str = "miles-weights", buffer_bytes: int = 512 << 20,
                 backend: Optional[str] = None, master_address: str = "127.0.0.1", master_port: Optional[int] = None,
                 engine_world_sizes: Optional[Sequence[int]] = None, is_sender: bool = True):
        # with an expert-parallel trainer every rank builds an updater (the expert gather is a collective of the
        # trainer's own group) but only the sender talks to the engines
        self.is_sender = is_sender
        self._base_name, self._generation = group_name, 0
        self.actor, self.engines, self.group_name = actor, list(engines), group_name
        self.buffer_bytes = buffer_bytes
        self.backend = backend or ("nccl" if actor.on_gpu else "gloo")
        self.master_address, self.master_port = master_address, master_port
        self.sizes = list(engine_world_sizes) if engine_world_sizes else [1] * len(self.engines)
        self.connected = False

    def connect(self) -> None:
        import socket

        if self.master_port is None:
            with socket.socket() as s:
                s.bind(("", 0))
                self.master_port = s.getsockname()[1]
        world = 1 + sum(self.sizes)
        handles, off = [], 1
        for e, n in zip(self.engines, self.sizes):
            handles.append(e.post_async("/init_weights_update_group", {
                "master_address": self.master_address, "master_port": self.master_port, "rank_offset": off,
                "world_size": world, "group_name": self.group_name, "backend": self.backend}))
            off += n
        init_update_group(self.master_address, self.master_port, 0, world, self.group_name, self.backend)
        for h in handles:
            h.result()
        self.connected = True

    def disconnect(self, skip: Sequence[int] = ()) -> None:
        for i, e in enumerate(self.engines):
            if i in skip:
                continue
            try:
                e.post("/destroy_weights_update_group", {"group_name": self.group_name})
            except Exception:
                pass  # an engine that is gone has no group left to destroy
        destroy_update_group(self.group_name)
        self.connected = False

    def replace_engine(self, index: int, engine) -> None:
        """A recovered engine took the place of a dead one: the old group (which still counts the dead process) is
        dropped and the next update builds a new one, under a new name and port, with the current engines."""
        if self.connected:
            self.disconnect(skip=(index,))
        self.engines[index] = engine
        self._generation += 1
        self.group_name = f"{self._base_name}-g{self._generation}"
        self.master_port = None

    def _named(self):
        store = self.actor.store
        dense = [(n, p) for n, p in store.params.items() if store.by_name[n].group == "dense"]
        experts = [(n, p) for n, p in store.params.items() if store.by_name[n].group == "expert"]
        if experts and store.ep_size > 1:
            gathered = []
            for n, p in experts:
                full = torch.empty((p.shape[0] * store.ep_size,) + tuple(p.shape[1:]), dtype=p.dtype, device=p.device)
                dist.all_gather_into_tensor(full, p.contiguous(), group=self.actor.ps.ep.group)
                gathered.append((n, full))
            experts = gathered
        return dense, experts

    def _parts(self):
        """Lists of ``(name, tensor)`` to send one after the other; a list's tensors stay valid until the next one is asked
        for. An unsharded store gives two (non-expert pass, expert pass); a sharded (``--train-backend fsdp``) store gives
        one per unit, whose parameters exist only while the unit is materialised (collective over the shard group: every
        trainer rank walks the units, the sender alone broadcasts them)."""
        store = self.actor.store
        if getattr(store, "is_fsdp", False):
            store.invalidate()
            for u in store.units:
                yield [(sp.name, store.params[sp.name]) for sp in u.specs]
            store.invalidate()
            return
        dense, experts = self._named()
        yield dense
        yield experts

    def update(self) -> dict:
        import time

        if not self.is_sender:
            for _ in self._parts():  # take part in the gathers, send nothing
                pass
            return {}
        if not self.connected:
            self.connect()
        t0 = time.perf_counter()
        mode = getattr(self.actor.args, "pause_generation_mode", "retract")
        for e in self.engines:
            e.post("/pause_generation", {"mode": mode})
            if mode != "in_place":
                e.post("/flush_cache", {})
        version = self.actor.store.version
        moved = 0
        for part in self._parts():
            for bucket in iter_buckets(part, self.buffer_bytes):
                hdr = bucket_header(bucket, self.group_name)
                handles = [e.post_async("/update_weights_from_distributed", hdr) for e in self.engines]
                moved += send_bucket(bucket, self.group_name)
                for h in handles:
                    h.result()
        for e in self.engines:
            e.post("/update_weight_version", {"new_version": version})
            e.post("/continue_generation", {})
        return {"perf/update_weights_time": time.perf_counter() - t0, "perf/update_weights_bytes": moved, "weight_version": version}


class HttpEngineHandle:
    """What ``BroadcastWeightUpdater`` needs from an engine in another process: blocking and background POSTs to its
    HTTP surface (`engine/server.py`). Background requests run on a small thread pool, because the engine answers
    ``/init_weights_update_group`` and ``/update_weights_from_distributed`` only once the trainer's side of the
    collective has started."""

    def __init__(self, base_url: str, timeout_s: float = 300.0, workers: int = 2):
        from concurrent.futures import ThreadPoolExecutor

        self.base = base_url.rstrip("/")
        self.timeout_s = timeout_s
        self._pool = ThreadPoolExecutor(max_workers=workers)

    def post(self, path: str, payload: Optional[dict] = None) -> dict:
        import json
        import urllib.request

        req = urllib.request.Request(self.base + path, data=json.dumps(payload or {}).encode(),
                                     headers={"Content-Type": "application/json"}, method="POST")
        with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
            body = r.read().decode()
        return json.loads(body) if body else {}

    def post_async(self, path: str, payload: Optional[dict] = None):
        return self._pool.submit(self.post, path, payload)

    def get(self, path: str) -> dict:
        import json
        import urllib.request

        with urllib.request.urlopen(self.base + path, timeout=self.timeout_s) as r:
            return json.loads(r.read().decode())

    def close(self) -> None:
        self._pool.shutdown(wait=False)
