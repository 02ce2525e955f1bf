"""In-process rollout engine: paged KV cache, continuous batching, CUDA-graph decode, sampling.

The engine owns no weights of its own: it runs the same model object (and therefore the same kernels
and the same parameter memory) as the trainer when colocated, which makes the trainer -> rollout weight
update a version bump.  It honours the contract the reference expects from its SGLang server
(miles/backends/sglang_utils/sglang_engine.py:126-693 and
miles/rollout/generate_utils/generate_endpoint_utils.py:52-140): token-in / token-out generation with
temperature / top-p / top-k / seed, stop tokens and max length, per-token log-probs of the sampled
tokens under the same temperature, finish reason ``stop | length | abort``, the weight version(s) a
sample was generated under, optional per-token routed experts (rollout routing replay), abort, pause /
continue, cache flush and memory release / resume.
"""
from __future__ import annotations

import itertools
import time
import zlib
from collections import deque
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..models.torch_impl import InferMeta


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    max_new_tokens: int = 128
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    sampling_seed: Optional[int] = None
    min_new_tokens: int = 0
    # benchmark hook (reference: rollout/generate_hub/benchmarkers.py): stop exactly at this length
    forced_length: Optional[int] = None

    # parameters of the reference's engines that would change what is sampled and are not built here: a request that sets
    # one to anything but its neutral value is refused instead of being served from another distribution
    UNSUPPORTED = {"min_p": 0.0, "repetition_penalty": 1.0, "frequency_penalty": 0.0, "presence_penalty": 0.0, "logit_bias": None,
                   "regex": None, "json_schema": None, "ebnf": None, "structural_tag": None, "n": 1}

    @classmethod
    def from_dict(cls, d: dict) -> "SamplingParams":
        d = dict(d or {})
        for k, neutral in cls.UNSUPPORTED.items():
            if d.get(k) not in (None, neutral):
                raise ValueError(f"sampling parameter {k}={d[k]!r} is not built in this engine (only its neutral value {neutral!r} is accepted)")
        stop = d.pop("stop_token_ids", None) or ()
        kw = {k: v for k, v in d.items() if k in cls.__dataclass_fields__}
        return cls(stop_token_ids=tuple(stop), **kw)


@dataclass
class Request:
    rid: str
    input_ids: list
    params: SamplingParams
    return_routed_experts: bool = False
    output_ids: list = field(default_factory=list)
    output_logprobs: list = field(default_factory=list)
    routed_experts: list = field(default_factory=list)  # per token [L, K] int32 cpu tensors
    weight_versions: list = field(default_factory=list)
    finish_reason: Optional[str] = None
    pages: list = field(default_factory=list)
    slot: int = -1  # row in the running batch
    seed: int = 0
    nodes: list = field(default_factory=list)  # prefix-cache nodes behind the first len(nodes) pages (shared, read only)
    prefill_cached: int = 0                    # tokens of the current prefill that came from the prefix cache
    cache_epoch: int = -1
    routes_tokens: int = 0                     # token positions covered by routed_experts so far
    t_submit: float = 0.0
    cached_tokens: int = 0

    @property
    def seq_len(self) -> int:
        return len(self.input_ids) + len(self.output_ids)

    def result(self) -> dict:
        """Response in the shape of the reference's /generate endpoint."""
        meta = {
            "output_token_logprobs": [(lp, tok) for lp, tok in zip(self.output_logprobs, self.output_ids)],
            "finish_reason": {"type": self.finish_reason or "abort"},
            "weight_version": self.weight_versions[-1] if self.weight_versions else 0,
            "weight_versions": list(self.weight_versions),
            "prompt_tokens": len(self.input_ids),
            "completion_tokens": len(self.output_ids),
            "cached_tokens": self.cached_tokens,
            "id": self.rid,
        }
        if self.return_routed_experts and self.routed_experts:
            meta["routed_experts"] = torch.cat(self.routed_experts, 0)
        return {"output_ids": list(self.output_ids), "meta_info": meta}


def _common_pages(a: list, b: list, ps: int, limit: int) -> int:
    """Number of leading full pages (of ``ps`` tokens, within the first ``limit`` tokens of ``a``) on which two token
    lists agree."""
    n = min(limit, len(b)) // ps
    k = 0
    while k < n and a[k * ps:(k + 1) * ps] == b[k * ps:(k + 1) * ps]:
        k += 1
    return k


def PagePool(num_pages: int):
    """KV page pool: the C++ free-list allocator of ``csrc/native/engine_core.cpp`` (page 0 is reserved as the
    dummy page of padded batch rows; ``alloc(n)`` returns a list of page ids or ``None``, ``release(pages)``,
    ``num_free``)."""
    from ..ops import _native

    return _native.load().PagePool(int(num_pages))


class Engine:
    def __init__(self, model, *, max_running: int = 64, num_pages: Optional[int] = None, page_size: int = 64,
                 max_seq_len: int = 16384, max_prefill_tokens: int = 16384, kv_mem_bytes: Optional[int] = None,
                 use_cuda_graph: Optional[bool] = None, eos_token_id: Optional[int] = None, kv_dtype=None,
                 sync=None, ep_decode=None, kv_storage: Optional[torch.Tensor] = None, overlap_decode: bool = True,
                 prefix_cache: bool = False, memory_saver: bool = False):
        self.model = model
        # KV cache in the tagged virtual-memory arena (utils/memory_saver.py): releasing it gives the physical memory
        # back but keeps the addresses, so captured decode graphs survive a release / resume cycle
        self._saver = None
        self._kv_tag = f"kv_cache_{id(self):x}"
        self._kv_paused = False
        if memory_saver and kv_storage is None and model.store.device.type == "cuda":
            from ..utils.memory_saver import MemorySaver

            saver = MemorySaver()
            self._saver = saver if saver.available else None
        self.prefix = None
        if prefix_cache:
            from .prefix_cache import PrefixCache

            self.prefix = PrefixCache(page_size)
        self.overlap_decode = overlap_decode  # keep one decode step in flight while the host reads the previous one
        self.kv_storage = kv_storage  # caller-owned uint8 device buffer to carve the KV cache from (None = allocate)
        # mixed into the sampling seed of requests that bring none: the loop sets it from --seed and the rank, so that a run
        # is reproducible, runs with different seeds differ, and the engines of different ranks do not sample in step
        self.seed_salt = 0
        self.sync = sync            # lockstep agreement across expert-parallel ranks (None = independent engine)
        self.ep_decode = ep_decode  # small expert-parallel exchange used by decode steps (graph friendly)
        self.last_mode = 0
        self._graph_pool = None
        self.cfg = model.cfg
        self.store = model.store
        self.dev = self.store.device
        self.on_gpu = self.dev.type == "cuda"
        self.page_size = page_size
        self.max_running = max_running
        self.max_seq_len = max_seq_len
        self.max_pages_per_seq = (max_seq_len + page_size - 1) // page_size
        self.max_prefill_tokens = max_prefill_tokens
        self.eos_token_id = eos_token_id
        self.kv_dtype = kv_dtype or self.store.dtype
        cfg = self.cfg
        per_page = 2 * cfg.num_layers * page_size * cfg.num_kv_heads * cfg.head_dim * torch.empty((), dtype=self.kv_dtype).element_size()
        if num_pages is None:
            if kv_mem_bytes is None:
                kv_mem_bytes = max_running * max_seq_len * per_page // page_size
            num_pages = max(2, kv_mem_bytes // per_page)
        self.num_pages = int(num_pages)
        self.pool = PagePool(self.num_pages)
        self.kv_cache: Optional[list] = None
        self._alloc_kv()
        self.waiting: deque = deque()
        self.running: list = []
        self.finished: dict = {}
        self.paused = False
        self.weight_version = 0
        self._rid = itertools.count()
        self.use_cuda_graph = self.on_gpu if use_cuda_graph is None else use_cuda_graph
        self._graphs: dict = {}
        self._alloc_decode_buffers()
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "decode_steps": 0, "retracted": 0}
        # host wall time and count of decode iterations per row bucket (the GPU is the bottleneck of a decode
        # iteration, so this is the step latency by batch size): {bucket: [seconds, steps]}
        self.bucket_time: dict = {}
        self._t_last_decode = None
        self.d2h_bytes = 0  # bytes read back from the device (sampled tokens, log-probs, routing)
        self.h2d_bytes = 0

    # ------------------------------------------------------------------ memory
    def _alloc_kv(self) -> None:
        cfg = self.cfg
        slots = self.num_pages * self.page_size
        if self.kv_storage is not None:
            # The buffer is shared in time with another user (the trainer's expert gradients): its contents
            # are undefined whenever a rollout starts, which is fine because every page is written by a
            # prefill or decode step before any position of it is read.
            per = slots * cfg.num_kv_heads * cfg.head_dim
            esz = torch.empty((), dtype=self.kv_dtype).element_size()
            assert self.kv_storage.numel() >= 2 * cfg.num_layers * per * esz, "kv_storage is too small"
            flat = self.kv_storage[:2 * cfg.num_layers * per * esz].view(self.kv_dtype)
            views = [flat[i * per:(i + 1) * per].view(slots, cfg.num_kv_heads, cfg.head_dim) for i in range(2 * cfg.num_layers)]
            self.kv_cache = [(views[2 * i], views[2 * i + 1]) for i in range(cfg.num_layers)]
            return
        import contextlib

        with (self._saver.region(self._kv_tag) if self._saver is not None else contextlib.nullcontext()):
            self.kv_cache = [(torch.zeros(slots, cfg.num_kv_heads, cfg.head_dim, dtype=self.kv_dtype, device=self.dev),
                              torch.zeros(slots, cfg.num_kv_heads, cfg.head_dim, dtype=self.kv_dtype, device=self.dev))
                             for _ in range(cfg.num_layers)]

    def _alloc_decode_buffers(self) -> None:
        B, dev = self.max_running, self.dev
        i32 = dict(dtype=torch.int32, device=dev)
        self.d_tokens = torch.zeros(B, **i32)
        self.d_positions = torch.zeros(B, **i32)
        self.d_seq_lens = torch.ones(B, **i32)
        self.d_slots = torch.zeros(B, **i32)
        self.d_block_table = torch.zeros(B, self.max_pages_per_seq, **i32)
        self.d_temperature = torch.ones(B, dtype=torch.float32, device=dev)
        self.d_top_k = torch.zeros(B, **i32)
        self.d_top_p = torch.ones(B, dtype=torch.float32, device=dev)
        self.d_seeds = torch.zeros(B, dtype=torch.int64, device=dev)
        self.d_step = torch.zeros(B, **i32)
        self.d_active = torch.zeros(B, **i32)
        self._rows: list = []
        self._rows_B = 0
        self.d_out_tokens = torch.zeros(B, **i32)
        self.d_out_logprobs = torch.zeros(B, dtype=torch.float32, device=dev)
        self.slots_free = list(range(B - 1, -1, -1))
        self.slot_req: list = [None] * B
        pin = self.on_gpu
        # two generations of result buffers: one decode step may be in flight while the previous one is read
        self.h_out = torch.zeros(2, B, dtype=torch.int32, pin_memory=pin)
        self.h_lp = torch.zeros(2, B, dtype=torch.float32, pin_memory=pin)
        self._h_routes: list = [None, None]
        self._parity = 0
        self._pending: Optional[dict] = None

    def release_memory_occupation(self, tags: Sequence[str] = ("kv_cache", "cuda_graph")) -> None:
        """Free the KV cache and/or captured graphs (weights are shared with the trainer and stay)."""
        self._drain_pending()
        assert not self.running, "release_memory_occupation with running requests; pause/abort first"
        if "cuda_graph" in tags:
            self._graphs.clear()
        if "kv_cache" in tags:
            if self.prefix is not None:
                self.pool.release(self.prefix.clear())  # the cached keys / values are gone with the memory
            if self._saver is not None and self.kv_cache is not None:
                if not self._kv_paused:
                    torch.cuda.synchronize(self.dev)
                    self._saver.pause(self._kv_tag)  # physical memory released, addresses (and graphs) stay valid
                    self._kv_paused = True
            else:
                self.kv_cache = None
                self._graphs.clear()  # graphs hold raw cache pointers
        if self.on_gpu:
            torch.cuda.empty_cache()

    def resume_memory_occupation(self, tags: Sequence[str] = ("kv_cache",)) -> None:
        if "kv_cache" in tags and self._kv_paused:
            self._saver.resume(self._kv_tag)
            self._kv_paused = False
            self.pool = PagePool(self.num_pages)
        elif "kv_cache" in tags and self.kv_cache is None:
            self._alloc_kv()
            self.pool = PagePool(self.num_pages)

    def flush_cache(self) -> bool:
        if self.running:
            if self.prefix is not None:
                # requests in flight keep the pages they use; everything else is forgotten (weights changed)
                self.pool.release(self.prefix.clear())
            return False
        self.pool = PagePool(self.num_pages)
        if self.prefix is not None:
            self.prefix.clear()
        return True

    # ------------------------------------------------------------------ prefill / decode disaggregation
    @torch.no_grad()
    def export_prefix(self, tokens: Sequence[int], to_cpu: bool = True) -> Optional[dict]:
        """The keys / values this engine's prefix cache holds for the longest cached prefix of ``tokens`` (whole pages):
        what a prefill engine hands to the decode engine that continues the request. ``kv`` is
        ``[layers, 2, cached_tokens, kv_heads, head_dim]``. None when nothing is cached."""
        if self.prefix is None or self.kv_cache is None or self._kv_paused:
            return None
        self._drain_pending()
        nodes = self.prefix.match([int(t) for t in tokens])
        if not nodes:
            return None
        ps = self.page_size
        pages = torch.tensor([n.page for n in nodes], dtype=torch.int64, device=self.dev)
        slots = (pages[:, None] * ps + torch.arange(ps, device=self.dev)[None, :]).reshape(-1)
        kv = torch.stack([torch.stack((kc[slots], vc[slots])) for kc, vc in self.kv_cache])
        payloads = [n.payload for n in nodes]
        return {"tokens": [int(t) for t in tokens[:len(nodes) * ps]], "kv": kv.cpu() if to_cpu else kv, "page_size": ps,
                "weight_version": self.weight_version,
                "routed_experts": torch.cat(payloads, 0).cpu() if all(p is not None for p in payloads) else None}

    @torch.no_grad()
    def import_prefix(self, blob: Optional[dict]) -> int:
        """Put exported keys / values into this engine's prefix cache, so that a request starting with those tokens
        prefills only what follows them. Pages already cached here are kept as they are. Returns the number of tokens the
        cache now holds for the sequence (0: refused because the page size or the weight version differs, the cache is off,
        or the pool has no room)."""
        if (blob is None or self.prefix is None or self.kv_cache is None or self._kv_paused
                or int(blob["page_size"]) != self.page_size or int(blob["weight_version"]) != self.weight_version):
            return 0
        self._drain_pending()
        ps = self.page_size
        tokens = [int(t) for t in blob["tokens"]]
        n_pages = len(tokens) // ps
        kv = blob["kv"]
        assert kv.shape[0] == len(self.kv_cache) and kv.shape[2] >= n_pages * ps, "exported keys / values of another model"
        have = self.prefix.match(tokens)
        self.prefix.lock(have)  # an eviction for the new pages must not take the pages we build upon
        try:
            need = n_pages - len(have)
            if need <= 0:
                return n_pages * ps
            new_pages = self._alloc(need)
            if new_pages is None:
                return len(have) * ps
            pg = torch.as_tensor(list(new_pages), dtype=torch.int64, device=self.dev)
            slots = (pg[:, None] * ps + torch.arange(ps, device=self.dev)[None, :]).reshape(-1)
            a = len(have) * ps
            part = kv[:, :, a:n_pages * ps].to(self.dev)
            for layer, (kc, vc) in enumerate(self.kv_cache):
                kc[slots] = part[layer, 0].to(kc.dtype)
                vc[slots] = part[layer, 1].to(vc.dtype)
            payloads = None
            if blob.get("routed_experts") is not None:
                re = blob["routed_experts"]
                payloads = [re[p * ps:(p + 1) * ps].clone() for p in range(n_pages)]
            nodes, dup = self.prefix.insert(tokens, [n.page for n in have] + list(new_pages), payloads, skip=len(have))
            if dup:
                self.pool.release(dup)
            return len(nodes) * ps
        finally:
            freed = self.prefix.unlock(have)
            if freed:
                self.pool.release(freed)

    def _alloc(self, n: int):
        """``n`` pages from the pool; when it runs dry, unreferenced prefix-cache pages are evicted first."""
        pages = self.pool.alloc(n)
        if pages is None and self.prefix is not None and self.prefix.num_pages:
            freed = self.prefix.evict(n - self.pool.num_free)
            if freed:
                self.pool.release(freed)
                pages = self.pool.alloc(n)
        return pages

    # ------------------------------------------------------------------ request API
    def add_request(self, input_ids: Sequence[int], params: SamplingParams | dict | None = None, rid: Optional[str] = None,
                    return_routed_experts: bool = False) -> str:
        if not isinstance(params, SamplingParams):
            params = SamplingParams.from_dict(params or {})
        rid = rid if rid is not None else f"req-{next(self._rid)}"
        ids = [int(t) for t in input_ids]
        if len(ids) + 1 > self.max_seq_len:
            ids = ids[-(self.max_seq_len - 1):]
        req = Request(rid, ids, params, return_routed_experts)
        req.seed = params.sampling_seed if params.sampling_seed is not None else (zlib.crc32(f"{self.seed_salt}:{rid}".encode()) & 0x7FFFFFFF)
        req.t_submit = time.time()
        self.waiting.append(req)
        return rid

    def abort_request(self, rid: Optional[str] = None, abort_all: bool = False) -> int:
        self._drain_pending()
        n = 0
        for req in list(self.running):
            if abort_all or req.rid == rid:
                self._finish(req, "abort")
                n += 1
        for req in list(self.waiting):
            if abort_all or req.rid == rid:
                self.waiting.remove(req)
                req.finish_reason = "abort"
                self.finished[req.rid] = req
                n += 1
        return n

    def pause_generation(self, mode: str = "retract") -> None:
        """``abort``: finish everything as aborted; ``retract``: running requests go back to the queue and
        will be re-prefilled (their generated tokens are kept); ``in_place``: keep KV and resume as is."""
        self._drain_pending()
        self.paused = True
        if mode == "abort":
            self.abort_request(abort_all=True)
        elif mode == "retract":
            for req in list(self.running):
                self._retract(req)

    def continue_generation(self) -> None:
        self.paused = False

    def update_weight_version(self, version: Optional[int] = None) -> int:
        self.weight_version = self.weight_version + 1 if version is None else int(version)
        return self.weight_version

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._pending is not None)

    def pop_finished(self) -> list:
        out = list(self.finished.values())
        self.finished.clear()
        return out

    # ------------------------------------------------------------------ scheduling
    def _pages_needed(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def _retract(self, req: Request) -> None:
        self._release(req, offer=True)
        self.running.remove(req)
        self.waiting.appendleft(req)
        self.stats["retracted"] += 1

    def _release(self, req: Request, offer: bool = False) -> None:
        """Give the request's pages back. ``offer``: its full pages (prompt and generated tokens) are offered to the
        prefix cache first, so a follow-up request that starts with this conversation finds them."""
        if req.pages:
            own = req.pages[len(req.nodes):]
            if self.prefix is not None:
                if offer and req.cache_epoch == self.prefix.epoch:
                    ids = req.input_ids + req.output_ids
                    # the last sampled token was never fed: keys / values exist for len(ids) - 1 positions
                    ids = ids[:len(ids) - 1]
                    payloads = self._page_payloads(req, len(ids) // self.page_size)
                    taken, dup = self.prefix.insert(ids, req.pages, payloads, skip=len(req.nodes))
                    keep = {n.page for n in taken[len(req.nodes):]}
                    own = [p for p in own if p not in keep or p in dup]
                own = own + self.prefix.unlock(req.nodes)
                req.nodes = []
            if own:
                self.pool.release(own)
            req.pages = []
        if req.slot >= 0:
            self.slot_req[req.slot] = None
            self.slots_free.append(req.slot)
            req.slot = -1

    def _page_payloads(self, req: Request, n_pages: int):
        """Routed experts of the request's first ``n_pages`` full pages (what routing replay needs when a later request
        takes those pages from the prefix cache), or None when the request did not record them."""
        if not (req.return_routed_experts and self.cfg.is_moe and req.routed_experts):
            return None
        allr = torch.cat(req.routed_experts, 0)
        ps = self.page_size
        return [allr[p * ps:(p + 1) * ps].clone() if (p + 1) * ps <= allr.shape[0] else None for p in range(n_pages)]

    def _finish(self, req: Request, reason: str) -> None:
        req.finish_reason = reason
        self._release(req, offer=True)
        if req in self.running:
            self.running.remove(req)
        self.finished[req.rid] = req

    def _check_stop(self, req: Request, tok: int) -> Optional[str]:
        p = req.params
        n = len(req.output_ids)
        if p.forced_length is not None:
            return "length" if n >= min(p.forced_length, p.max_new_tokens) else None
        if n >= p.min_new_tokens and not p.ignore_eos:
            if tok in p.stop_token_ids or (self.eos_token_id is not None and tok == self.eos_token_id):
                return "stop"
        if n >= p.max_new_tokens or req.seq_len >= self.max_seq_len:
            return "length"
        return None

    def step(self) -> list:
        """One scheduler iteration: a prefill batch if requests can be admitted, else one decode step.

        With ``sync`` every expert-parallel rank agrees on the kind of iteration (2 prefill, 1 decode, 0 idle);
        ranks without matching work run a one-token dummy forward so that the MoE exchanges stay aligned."""
        if self.kv_cache is None or self._kv_paused:
            return []
        before = set(self.finished)
        admitted = [] if self.paused else self._admit()
        local = 2 if admitted else (1 if ((self.running and not self.paused) or self._pending is not None) else 0)
        bucket = None
        if self.sync is not None:
            # one host agreement per iteration: the kind of iteration and, for a decode step, the row bound every rank
            # pads its batch to (the expert-parallel exchange needs the same bound everywhere)
            want = self._bucket(max(len(self.running), 1)) if (local == 1 and not self.paused) else 0
            mode, bucket = self.sync.agree(local, want)
            bucket = max(bucket, 1)
        else:
            mode = local
        self.last_mode = mode
        if mode == 2:
            self._prefill(admitted)
        elif mode == 1:
            if self.sync is not None:
                self._decode_lockstep(bucket)
            else:
                self._decode()
        return [self.finished[r] for r in self.finished if r not in before]

    def drain(self) -> None:
        """Keep stepping (with dummy work) until every rank of the lockstep group is idle."""
        if self.sync is None:
            return
        while True:
            self.step()
            if self.last_mode == 0:
                break

    def _admit(self) -> list:
        batch, tokens = [], 0
        if self.prefix is None:
            while self.waiting and self.slots_free:
                req = self.waiting[0]
                n = req.seq_len
                if batch and tokens + n > self.max_prefill_tokens:
                    break
                pages = self._alloc(self._pages_needed(n + 1))
                if pages is None:
                    break
                self.waiting.popleft()
                req.pages = pages
                req.slot = self.slots_free.pop()
                self.slot_req[req.slot] = req
                batch.append(req)
                tokens += n
            return batch
        # with a prefix cache: a request that shares more full pages with one admitted in this very batch than the cache
        # holds yet is left for the next iteration, when those pages exist (the samples of one prompt then compute the
        # prompt once); the others keep their order
        ps = self.page_size
        admitted_ids: list = []
        for req in list(self.waiting):
            if not self.slots_free:
                break
            ids = req.input_ids + req.output_ids
            n = len(ids)
            nodes = self.prefix.match(ids, n - 1, need_payload=req.return_routed_experts and self.cfg.is_moe)
            if any(_common_pages(ids, other, ps, n - 1) > len(nodes) for other in admitted_ids):
                continue
            new_tokens = n - len(nodes) * ps
            if batch and tokens + new_tokens > self.max_prefill_tokens:
                break
            self.prefix.lock(nodes)  # before allocating: the eviction that may run now must not take them
            pages = self._alloc(self._pages_needed(n + 1) - len(nodes))
            if pages is None:
                self.pool.release(self.prefix.unlock(nodes))
                break
            self.waiting.remove(req)
            req.nodes, req.pages = list(nodes), [nd.page for nd in nodes] + pages
            req.prefill_cached, req.cache_epoch = len(nodes) * ps, self.prefix.epoch
            req.cached_tokens += req.prefill_cached  # reported as meta_info.cached_tokens
            if req.return_routed_experts and self.cfg.is_moe and req.routes_tokens < req.prefill_cached:
                req.routed_experts = [nd.payload for nd in nodes]
                req.routes_tokens = req.prefill_cached
            req.slot = self.slots_free.pop()
            self.slot_req[req.slot] = req
            batch.append(req)
            admitted_ids.append(ids)
            tokens += new_tokens
        return batch

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def _prefill(self, batch: list) -> None:
        dev, ps = self.dev, self.page_size
        toks, pos, slots, cu = [], [], [], [0]
        if not batch:  # lockstep dummy: one token written to the reserved page 0
            toks, pos, slots, cu = [0], [0], [torch.zeros(1, dtype=torch.int64)], [0, 1]
        prefix_lens, pre_slots = [], []
        for req in batch:
            ids = req.input_ids + req.output_ids
            n, c = len(ids), req.prefill_cached
            toks.extend(ids[c:])
            pos.extend(range(c, n))
            pg = torch.tensor(req.pages, dtype=torch.int64)
            idx = torch.arange(n)
            sl = pg[idx // ps] * ps + idx % ps
            slots.append(sl[c:])
            pre_slots.append(sl[:c])
            prefix_lens.append(c)
            cu.append(cu[-1] + n - c)
        # one pinned host staging buffer per prefill: tokens | positions | slot mapping | cu_seqlens, one H2D copy
        n_tok = len(toks)
        host = torch.empty(3 * n_tok + len(cu), dtype=torch.int32, pin_memory=self.on_gpu)
        host[:n_tok] = torch.tensor(toks, dtype=torch.int32)
        host[n_tok:2 * n_tok] = torch.tensor(pos, dtype=torch.int32)
        host[2 * n_tok:3 * n_tok] = torch.cat(slots).to(torch.int32)
        host[3 * n_tok:] = torch.tensor(cu, dtype=torch.int32)
        staged = host.to(dev, non_blocking=True)
        tokens, positions, slot_mapping, cu_t = (staged[:n_tok], staged[n_tok:2 * n_tok], staged[2 * n_tok:3 * n_tok],
                                                 staged[3 * n_tok:])
        max_len = max(b - a for a, b in zip(cu[:-1], cu[1:]))
        meta = InferMeta(True, cu_t, max_len, slot_mapping, page_size=ps)
        if any(prefix_lens):
            # part of every sequence is already in the KV cache: the attention reads those keys / values from their
            # pages (prefix slots) next to the ones this pass computes
            from ..models.torch_impl import PrefixInfo

            meta.prefix = PrefixInfo.build(prefix_lens, [b - a for a, b in zip(cu[:-1], cu[1:])], torch.cat(pre_slots), dev)
            self.stats["cached_tokens"] = self.stats.get("cached_tokens", 0) + sum(prefix_lens)
        want_routes = any(r.return_routed_experts for r in batch) and self.cfg.is_moe
        record = [] if want_routes else None
        kw = {"max_seqlen": max_len} if self.on_gpu and hasattr(self.model, "launches") else {}
        h = self.model.forward_hidden(tokens, positions, cu_t, meta=meta, kv_cache=self.kv_cache, record=record, **kw)
        if not batch:
            return
        last = torch.tensor([c - 1 for c in cu[1:]], dtype=torch.int64, device=dev)
        logits = self.model.logits(h[last])
        tok, lp = self._sample(logits, batch)
        tok_l, lp_l = tok.tolist(), lp.tolist()
        routes = torch.stack(record, 1).cpu() if want_routes else None  # [T, L, K]
        self.d2h_bytes += 8 * len(batch) + (routes.numel() * 4 if routes is not None else 0)
        self.h2d_bytes += 12 * len(toks) + 4 * len(cu)
        self.stats["prefill_tokens"] += len(toks)
        for i, req in enumerate(batch):
            if routes is not None and req.return_routed_experts:
                # this pass covered positions [cached, n): keep what is not recorded yet (after a retraction only the
                # position of the token that had been sampled but not fed is new)
                n_i = req.prefill_cached + (cu[i + 1] - cu[i])
                start = max(req.routes_tokens, req.prefill_cached)
                if start < n_i:
                    req.routed_experts.append(routes[cu[i] + (start - req.prefill_cached):cu[i + 1]])
                    req.routes_tokens = n_i
            if self.prefix is not None and req.cache_epoch == self.prefix.epoch:
                # the full pages this pass completed join the prefix tree at once (the other samples of the prompt are
                # waiting for exactly these); the request keeps using them through references
                ids = req.input_ids + req.output_ids
                if len(ids) // ps > len(req.nodes):
                    nodes, _ = self.prefix.insert(ids, req.pages, self._page_payloads(req, len(ids) // ps), skip=len(req.nodes),
                                                  stop_at_duplicate=True)
                    self.prefix.lock(nodes[len(req.nodes):])
                    req.nodes = list(nodes)
            req.prefill_cached = 0
            self.running.append(req)
            self._append_token(req, int(tok_l[i]), float(lp_l[i]))

    def _sample(self, logits: torch.Tensor, reqs: list, steps: Optional[list] = None):
        """Eager sampling for a list of requests (prefill path). ``steps``: per-request sampling step counters (the
        number of tokens generated so far); decode passes the device-side counters because a look-ahead step runs
        before the host has appended the previous token."""
        n = len(reqs)
        if steps is None:
            steps = [len(r.output_ids) for r in reqs]
        if self.on_gpu and hasattr(self.model, "C"):
            dev = self.dev
            t = torch.tensor([r.params.temperature for r in reqs], dtype=torch.float32, device=dev)
            k = torch.tensor([r.params.top_k if r.params.top_k else 0 for r in reqs], dtype=torch.int32, device=dev)
            p = torch.tensor([r.params.top_p for r in reqs], dtype=torch.float32, device=dev)
            s = torch.tensor([r.seed for r in reqs], dtype=torch.int64, device=dev)
            st = torch.tensor(steps, dtype=torch.int32, device=dev)
            out = torch.empty(n, dtype=torch.int32, device=dev)
            lp = torch.empty(n, dtype=torch.float32, device=dev)
            self.model.C.sample_rows(logits, t, k, p, s, st, out, lp)
            self.model.launches += 1
            return out, lp
        from ..ops import reference as R

        toks, lps = [], []
        for i, r in enumerate(reqs):
            g = torch.Generator(device=logits.device).manual_seed((r.seed * 1000003 + int(steps[i])) & 0x7FFFFFFF)
            tk, l = R.sample(logits[i:i + 1], r.params.temperature, r.params.top_k, r.params.top_p, g)
            toks.append(tk)
            lps.append(l)
        return torch.cat(toks), torch.cat(lps)

    def _append_token(self, req: Request, tok: int, lp: float) -> None:
        req.output_ids.append(tok)
        req.output_logprobs.append(lp)
        if not req.weight_versions or req.weight_versions[-1] != self.weight_version:
            req.weight_versions.append(self.weight_version)
        reason = self._check_stop(req, tok)
        if reason:
            self._finish(req, reason)

    # ------------------------------------------------------------------ decode
    def _grow_pages(self) -> None:
        """Make sure every running request owns the page its next token is written to."""
        for req in list(self.running):
            if req not in self.running:  # retracted as a victim earlier in this pass
                continue
            need = self._pages_needed(req.seq_len)
            while len(req.pages) < need:
                pg = self._alloc(1)
                if pg is None:
                    victim = self.running[-1]
                    self._retract(victim)
                    if victim is req:
                        break
                    continue
                req.pages.extend(pg)

    def _bucket(self, n: int) -> int:
        b = 1
        while b < n:
            b *= 2
        if b > 16:
            b = (n + 15) // 16 * 16
        return min(max(b, 1), self.max_running)

    def _upload_rows(self, reqs: list, B: int) -> None:
        """Full refresh of the device-side decode state (only when the batch composition changed)."""
        W = self.max_pages_per_seq
        h_i = torch.zeros(B, 6 + W, dtype=torch.int32)  # tok, pos, len, top_k, step, active, block_table...
        h_i[:, 2] = 1
        h_f = torch.ones(B, 2, dtype=torch.float32)
        h_s = torch.zeros(B, dtype=torch.int64)
        for i, r in enumerate(reqs):
            L = r.seq_len  # tokens so far; the last one is the input of this step
            h_i[i, 0], h_i[i, 1], h_i[i, 2] = r.output_ids[-1], L - 1, L
            h_i[i, 3], h_i[i, 4], h_i[i, 5] = (r.params.top_k or 0), len(r.output_ids), 1
            h_i[i, 6:6 + len(r.pages)] = torch.tensor(r.pages, dtype=torch.int32)
            h_f[i, 0], h_f[i, 1] = r.params.temperature, r.params.top_p
            h_s[i] = r.seed
        d_i = h_i.to(self.dev, non_blocking=False)
        self.d_tokens[:B] = d_i[:, 0]
        self.d_positions[:B] = d_i[:, 1]
        self.d_seq_lens[:B] = d_i[:, 2]
        self.d_top_k[:B] = d_i[:, 3]
        self.d_step[:B] = d_i[:, 4]
        self.d_active[:B] = d_i[:, 5]
        self.d_block_table[:B] = d_i[:, 6:]
        d_f = h_f.to(self.dev)
        self.d_temperature[:B] = d_f[:, 0]
        self.d_top_p[:B] = d_f[:, 1]
        self.d_seeds[:B] = h_s.to(self.dev)
        for r in reqs:
            r.dev_pages = len(r.pages)
        self._rows = list(reqs)
        self._rows_B = B

    # ------------------------------------------------------------------ decode: launch / process, one step in flight
    def _grow_pages_ahead(self, lookahead: int) -> bool:
        """Pages for ``lookahead`` more positions of every running request, without retracting anybody.
        False if the pool cannot provide them (pages obtained so far stay with their requests)."""
        for req in self.running:
            need = self._pages_needed(req.seq_len + lookahead)
            while len(req.pages) < need:
                pg = self._alloc(1)
                if pg is None:
                    return False
                req.pages.extend(pg)
        return True

    @torch.no_grad()
    def _launch_decode(self, lookahead: int, bucket: Optional[int] = None) -> Optional[dict]:
        """Enqueue one decode step for the running set and the copies of its results into pinned host buffers.
        ``lookahead = 1``: the step *after* the one still in flight (same batch, device-side state already advances
        inside the captured step), launched before the host has looked at the previous step's tokens."""
        if lookahead == 0:
            self._grow_pages()
        elif not self._grow_pages_ahead(lookahead):
            return None
        reqs = list(self.running) if not self.paused else []
        if not reqs and self.sync is None:
            return None
        n = len(reqs)
        B = self._bucket(max(n, 1)) if bucket is None else max(int(bucket), self._bucket(max(n, 1)))
        same = (self._rows_B == B and len(self._rows) == n and all(a is b for a, b in zip(self._rows, reqs)))
        if not same:
            assert lookahead == 0, "a look-ahead step never changes the batch"
            self._upload_rows(reqs, B)
        else:
            for i, r in enumerate(reqs):  # pages appended since the device-side table was last written (wherever they
                for j in range(getattr(r, "dev_pages", 0), len(r.pages)):  # were obtained: here or by a look-ahead check)
                    self.d_block_table[i, j] = r.pages[j]
                r.dev_pages = len(r.pages)
        want_routes = self.cfg.is_moe and any(r.return_routed_experts for r in reqs)
        ll = getattr(self.ep_decode, "low_latency", False)
        if ll:
            # every rank replays the same graph for a row bound: routing is always recorded, padding rows are masked
            want_routes = self.cfg.is_moe
            self.ep_decode.set_step(B, self.d_active)
        saved_ep = getattr(self.model, "ep", None)
        if self.ep_decode is not None:
            self.model.ep = self.ep_decode
        try:
            routes = self._run_decode(B, want_routes)
        finally:
            if self.ep_decode is not None:
                self.model.ep = saved_ep
        if n == 0:
            return None
        par = self._parity
        self._parity ^= 1
        pend = {"reqs": reqs, "n": n, "parity": par, "event": None, "routes": None, "bucket": B}
        if self.on_gpu:
            self.h_out[par, :n].copy_(self.d_out_tokens[:n], non_blocking=True)
            self.h_lp[par, :n].copy_(self.d_out_logprobs[:n], non_blocking=True)
            if routes is not None:
                hr = self._h_routes[par]
                if hr is None or hr.shape[0] < n or hr.shape[1:] != routes.shape[1:]:
                    hr = torch.empty((self.max_running,) + tuple(routes.shape[1:]), dtype=routes.dtype, pin_memory=True)
                    self._h_routes[par] = hr
                hr[:n].copy_(routes[:n], non_blocking=True)
                pend["routes"] = hr
            ev = torch.cuda.Event()
            ev.record()
            pend["event"] = ev
        else:
            self.h_out[par, :n] = self.d_out_tokens[:n]
            self.h_lp[par, :n] = self.d_out_logprobs[:n]
            pend["routes"] = routes[:n].clone() if routes is not None else None
        return pend

    def _process_decode(self, pend: dict) -> None:
        """Read one step's sampled tokens on the host and advance the requests (a request that finished, was
        retracted or aborted after the step was launched ignores its row)."""
        if pend["event"] is not None:
            pend["event"].synchronize()
        now = time.perf_counter()
        if self._t_last_decode is not None and pend.get("bucket"):
            bt = self.bucket_time.setdefault(pend["bucket"], [0.0, 0])
            dt = now - self._t_last_decode
            if dt < 0.5:  # a gap that long is a prefill or an idle period, not a decode step
                bt[0] += dt
                bt[1] += 1
        self._t_last_decode = now
        n, par = pend["n"], pend["parity"]
        tok_l, lp_l = self.h_out[par, :n].tolist(), self.h_lp[par, :n].tolist()
        routes_c = pend["routes"]
        self.d2h_bytes += 8 * n + (routes_c[:n].numel() * 4 if routes_c is not None else 0)
        self.stats["decode_steps"] += 1
        for i, r in enumerate(pend["reqs"]):
            if r.finish_reason is not None or r.slot < 0:
                continue
            if routes_c is not None and r.return_routed_experts:
                r.routed_experts.append(routes_c[i:i + 1].clone())
                r.routes_tokens += 1
            self.stats["decode_tokens"] += 1
            self._append_token(r, int(tok_l[i]), float(lp_l[i]))

    def _can_look_ahead(self, pend: dict) -> bool:
        if not self.overlap_decode or self.sync is not None or self.paused or self.waiting:
            return False
        reqs = pend["reqs"]
        if len(reqs) != len(self.running) or any(a is not b for a, b in zip(reqs, self.running)):
            return False
        for r in reqs:  # a request that is certain to stop at the step in flight ends the speculation
            p = r.params
            limit = p.max_new_tokens if p.forced_length is None else min(p.forced_length, p.max_new_tokens)
            if len(r.output_ids) + 1 >= limit or r.seq_len + 2 >= self.max_seq_len:
                return False
        return True

    def _can_launch_ahead(self, pend: dict, bucket: int) -> bool:
        """Lockstep engines: may the next step be launched before the host has seen the step in flight? Only when
        nothing about the batch can change: same requests, same row bound, nobody certain to stop, pages at hand."""
        if not self.overlap_decode or self.paused or self.waiting or bucket != self._rows_B:
            return False
        reqs = pend["reqs"]
        if len(reqs) != len(self.running) or any(a is not b for a, b in zip(reqs, self.running)):
            return False
        for r in reqs:
            p = r.params
            limit = p.max_new_tokens if p.forced_length is None else min(p.forced_length, p.max_new_tokens)
            if len(r.output_ids) + 1 >= limit or r.seq_len + 2 >= self.max_seq_len:
                return False
        return self._grow_pages_ahead(1)

    @torch.no_grad()
    def _decode_lockstep(self, bucket: int) -> None:
        """One decode iteration of a lockstep (expert-parallel) engine: exactly one step is launched per call on
        every rank, with ``bucket`` rows (a rank without requests launches padding rows only), so that the ranks'
        exchanges stay aligned; the step launched by the previous call is read back after the new launch whenever
        the batch cannot have changed, which hides the host work and the agreement behind the GPU."""
        prev, self._pending = self._pending, None
        ahead = prev is not None and self._can_launch_ahead(prev, bucket)
        if prev is not None and not ahead:
            self._process_decode(prev)
            prev = None
        new = self._launch_decode(1 if ahead else 0, bucket=bucket)
        if prev is not None:
            self._process_decode(prev)
        self._pending = new

    def warm_up_decode_graphs(self) -> None:
        """Capture the decode graph of every row bound now (all ranks of a lockstep group call this at the same
        point): capturing runs a step twice, which a rank must not do on its own in the middle of a rollout."""
        if not (self.use_cuda_graph and self.on_gpu) or self.kv_cache is None:
            return
        buckets = sorted({self._bucket(n) for n in range(1, self.max_running + 1)})
        ll = getattr(self.ep_decode, "low_latency", False)
        saved_ep = getattr(self.model, "ep", None)
        for B in buckets:
            self._upload_rows([], B)
            if ll:
                self.ep_decode.set_step(B, self.d_active)
            if self.ep_decode is not None:
                self.model.ep = self.ep_decode
            try:
                self._run_decode(B, self.cfg.is_moe if ll else False)
            finally:
                if self.ep_decode is not None:
                    self.model.ep = saved_ep
        torch.cuda.synchronize()
        self._rows, self._rows_B = [], 0

    def _drain_pending(self) -> None:
        if self._pending is not None:
            pend, self._pending = self._pending, None
            self._process_decode(pend)

    @torch.no_grad()
    def _decode(self) -> None:
        """One decode step becomes visible to the host per call, while the next one is already running: the host
        work between steps (reading tokens, stop checks, page bookkeeping) no longer leaves the GPU idle."""
        pend, self._pending = self._pending, None
        if pend is None:
            pend = self._launch_decode(0)
            if pend is None:
                return
        nxt = self._launch_decode(1) if self._can_look_ahead(pend) else None
        self._process_decode(pend)
        self._pending = nxt

    def _decode_body(self, B: int, want_routes: bool):
        ps = self.page_size
        pos = self.d_positions[:B]
        page = self.d_block_table[:B].gather(1, (pos // ps).long()[:, None])[:, 0]
        self.d_slots[:B] = page * ps + pos % ps
        meta = InferMeta(False, None, 0, self.d_slots[:B], self.d_block_table[:B], self.d_seq_lens[:B], ps)
        record = [] if want_routes else None
        h = self.model.forward_hidden(self.d_tokens[:B], pos, None, meta=meta, kv_cache=self.kv_cache, record=record)
        logits = self.model.logits(h)
        if self.on_gpu and hasattr(self.model, "C"):
            self.model.C.sample_rows(logits, self.d_temperature[:B], self.d_top_k[:B], self.d_top_p[:B], self.d_seeds[:B],
                                     self.d_step[:B], self.d_out_tokens[:B], self.d_out_logprobs[:B])
            self.model.launches += 1
        else:
            reqs = list(self._rows)
            tok, lp = self._sample(logits[:len(reqs)], reqs, steps=self.d_step[:len(reqs)].tolist())
            self.d_out_tokens[:len(reqs)] = tok.to(torch.int32)
            self.d_out_logprobs[:len(reqs)] = lp
        # advance the device-side state so that the next step needs no host upload
        act = self.d_active[:B]
        self.d_tokens[:B] = torch.where(act > 0, self.d_out_tokens[:B], self.d_tokens[:B])
        self.d_positions[:B] += act
        self.d_seq_lens[:B] += act
        self.d_step[:B] += act
        return torch.stack(record, 1) if want_routes else None

    def _run_decode(self, B: int, want_routes: bool):
        if not (self.use_cuda_graph and self.on_gpu):
            return self._decode_body(B, want_routes)
        key = (B, want_routes)
        entry = self._graphs.get(key)
        if entry is None:
            # warm-up outside capture (first-use attribute setup, allocator growth), then capture
            launches0 = getattr(self.model, "launches", 0)
            self._decode_body(B, want_routes)
            torch.cuda.synchronize()
            per_replay = getattr(self.model, "launches", 0) - launches0
            g = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(g, pool=self._graph_pool):
                out = self._decode_body(B, want_routes)
            entry = (g, out, per_replay)
            self._graphs[key] = entry
            if hasattr(self.model, "launches"):
                self.model.launches -= 2 * per_replay  # neither the warm-up nor the capture pass produced tokens
            # the warm-up run advanced the device-side decode state; rewind it before the first real replay
            self._upload_rows(list(self._rows), B)
        g, out, per_replay = entry
        g.replay()
        if hasattr(self.model, "launches"):
            self.model.launches += per_replay
        return out

    # ------------------------------------------------------------------ scoring
    @torch.no_grad()
    def score(self, input_ids: Sequence[int], temperature: float = 1.0, top_k: int = 0) -> dict:
        """Log-probs this model gives to a token sequence (no generation, no KV cache): ``logprobs[i]`` is the log-prob
        of token ``i`` given the tokens before it (``None`` for the first). With ``top_k`` also the ``top_k`` most likely
        tokens and their log-probs at every position (``top[i]`` predicts token ``i``). The scoring endpoint of a
        teacher in on-policy distillation (``/generate`` with ``max_new_tokens = 0``)."""
        ids = [int(t) for t in input_ids]
        n = len(ids)
        if n < 2:
            return {"logprobs": [None] * n, "top": [None] * n}
        dev = self.dev
        tok = torch.tensor(ids, dtype=torch.int32, device=dev)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        cu = torch.tensor([0, n], dtype=torch.int32, device=dev)
        rows = torch.arange(0, n - 1, dtype=torch.int64, device=dev)
        kw = {"max_seqlen": n} if self.on_gpu and hasattr(self.model, "launches") else {}
        inv_t = 1.0 / max(float(temperature), 1e-6)
        top = [None] * n
        if top_k > 0:
            h = self.model.forward_hidden(tok, pos, cu, **kw)
            ls = torch.log_softmax(self.model.logits(h[rows]).float() * inv_t, dim=-1)
            lp = ls.gather(1, tok[1:].long()[:, None])[:, 0]
            tv, ti = ls.topk(min(top_k, ls.shape[1]), dim=-1)
            top = [None] + [{"ids": ti[i].tolist(), "logprobs": tv[i].tolist()} for i in range(n - 1)]
        else:
            lp, _ = self.model.forward_logprobs(tok, pos, cu, rows, tok[1:], inv_t, **kw)
        self.stats["scored_tokens"] = self.stats.get("scored_tokens", 0) + n
        return {"logprobs": [None] + [float(x) for x in lp.tolist()], "top": top}

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams] | dict | None = None,
                 return_routed_experts: bool = False) -> list:
        """Blocking batch generation: returns results in prompt order."""
        rids = []
        for i, p in enumerate(prompts):
            sp = params[i] if isinstance(params, (list, tuple)) else params
            rids.append(self.add_request(p, sp, return_routed_experts=return_routed_experts))
        done: dict = {}
        while self.has_work():
            if self.paused:
                raise RuntimeError("generate() called while generation is paused")
            for req in self.step():
                done[req.rid] = req
        for req in self.pop_finished():
            done.setdefault(req.rid, req)
        return [done[r].result() for r in rids]


class LockstepSync:
    """Agreement on the kind of engine iteration across expert-parallel ranks (MAX over a tiny CPU tensor)."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.buf = torch.zeros(2, dtype=torch.int32)

    def agree(self, mode: int, bucket: int = 0) -> tuple:
        """MAX over the ranks of (kind of iteration, rows wanted for a decode step)."""
        self.buf[0], self.buf[1] = mode, bucket
        self.dist.all_reduce(self.buf, op=self.dist.ReduceOp.MAX, group=self.group)
        return int(self.buf[0]), int(self.buf[1])
