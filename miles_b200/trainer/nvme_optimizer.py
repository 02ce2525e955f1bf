"""Adam whose states live in files: fp32 master parameters and both moments are stored per bucket on a local
disk (NVMe), and ``step()`` streams one bucket at a time through the device, so a model trains whose optimizer
states fit neither in device nor in host memory.

Per bucket (at most ``bucket_elems`` elements of a flat parameter buffer): read master / m / v from the bucket's
file into pinned staging buffers, copy to the device, run the fused Adam kernel on the bucket's slice of the live
bf16 parameters and gradients, copy the new states back and write them to the file. Reads of bucket ``i + 1`` are
issued on a worker thread while bucket ``i`` computes. Moments may be kept on disk in a narrower type
(``fp32`` / ``bf16`` / ``fp16``); the arithmetic is always fp32.

Reference: miles_plugins/optimizers/nvme_stream.py:1-522 (bucket size constant :47-58, on-disk dtypes).
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

_DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
_NP = {torch.float32: np.float32, torch.bfloat16: np.uint16, torch.float16: np.float16}


class NvmeStreamedAdam:
    def __init__(self, store, directory: str, lr: float = 1e-6, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, bucket_elems: int = 200_000_000, moment_dtype: str = "fp32",
                 clip_grad: float = 0.0):
        self.store, self.dir = store, directory
        self.lr, self.b1, self.b2, self.eps, self.wd = lr, betas[0], betas[1], eps, weight_decay
        self.clip_grad = clip_grad
        self.mdt = _DT[moment_dtype]
        self.step_count = 0
        self.dev = store.device
        os.makedirs(directory, exist_ok=True)
        self.buckets = []  # (group, start, end, path)
        for g, flat in store.flat.items():
            n = flat.numel()
            for i, a in enumerate(range(0, n, bucket_elems)):
                self.buckets.append((g, a, min(a + bucket_elems, n), os.path.join(directory, f"{g}_{i:05d}")))
        self._pool = ThreadPoolExecutor(max_workers=2)
        self.bytes_read = self.bytes_written = 0
        self._init_files()

    # ------------------------------------------------------------------ files
    def _paths(self, base: str) -> tuple:
        return base + ".master.bin", base + ".m.bin", base + ".v.bin"

    def _init_files(self) -> None:
        for g, a, b, base in self.buckets:
            pm, pmo, pv = self._paths(base)
            if all(os.path.exists(p) for p in (pm, pmo, pv)):
                continue
            self._write(pm, self.store.flat[g][a:b].detach().float().cpu())
            z = torch.zeros(b - a, dtype=self.mdt)
            self._write(pmo, z)
            self._write(pv, z)

    def _write(self, path: str, t: torch.Tensor) -> None:
        arr = t.contiguous().view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()
        tmp = path + ".tmp"
        arr.tofile(tmp)
        os.replace(tmp, path)
        self.bytes_written += arr.nbytes

    def _read(self, path: str, n: int, dtype: torch.dtype) -> torch.Tensor:
        arr = np.fromfile(path, dtype=_NP[dtype], count=n)
        self.bytes_read += arr.nbytes
        t = torch.from_numpy(arr)
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t

    def _load_bucket(self, k: int) -> tuple:
        g, a, b, base = self.buckets[k]
        pm, pmo, pv = self._paths(base)
        n = b - a
        return self._read(pm, n, torch.float32), self._read(pmo, n, self.mdt), self._read(pv, n, self.mdt)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def grad_norm(self) -> torch.Tensor:
        tot = torch.zeros((), dtype=torch.float32, device=self.dev)
        for g in self.store.grad.values():
            if g is not None and g.numel():
                tot += g.float().pow(2).sum()
        return tot.sqrt()

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        self.step_count += 1
        norm = self.grad_norm()
        scale = 1.0
        if self.clip_grad and self.clip_grad > 0:
            scale = float(torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0))
        bc1 = 1.0 - self.b1 ** self.step_count
        bc2 = 1.0 - self.b2 ** self.step_count
        nxt = self._pool.submit(self._load_bucket, 0) if self.buckets else None
        pending = []
        for k, (g, a, b, base) in enumerate(self.buckets):
            master, m, v = nxt.result()
            nxt = self._pool.submit(self._load_bucket, k + 1) if k + 1 < len(self.buckets) else None
            master, m, v = master.to(self.dev), m.to(self.dev).float(), v.to(self.dev).float()
            grad = self.store.grad[g][a:b].float() * scale
            m.mul_(self.b1).add_(grad, alpha=1.0 - self.b1)
            v.mul_(self.b2).addcmul_(grad, grad, value=1.0 - self.b2)
            upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
            if self.wd:
                upd.add_(master, alpha=self.wd)
            master.add_(upd, alpha=-self.lr)
            self.store.flat[g][a:b].copy_(master.to(self.store.flat[g].dtype))
            pm, pmo, pv = self._paths(base)
            for fut in pending:  # at most one bucket of writes in flight behind the compute
                fut.result()
            host = (master.cpu(), m.to(self.mdt).cpu(), v.to(self.mdt).cpu())
            pending = [self._pool.submit(self._write, p, t) for p, t in zip((pm, pmo, pv), host)]
        for fut in pending:
            fut.result()
        self.store.version += 1
        return norm

    def state_dict(self) -> dict:
        return {"step": self.step_count, "dir": self.dir, "moment_dtype": str(self.mdt)}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
