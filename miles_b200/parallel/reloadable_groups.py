"""Process groups that can be torn down and rebuilt between phases.

A NCCL communicator pins device memory (its channel buffers) for as long as it lives. A colocated trainer that sleeps
while the rollout engine runs can hand that memory over: ``release()`` destroys every sub-group created through
``new_group`` here, ``reload()`` creates them again in the same order on every rank. The world group stays (it bootstraps
the new ones).

Objects all over the trainer keep references to group objects (optimizers, dispatchers, stores). Instead of wrapping
every ``torch.distributed`` call so that it unwraps a proxy (what the reference does by patching ``torch.distributed``,
miles/utils/reloadable_process_group.py:13-282), the registry asks the garbage collector which dicts and lists hold a
group about to be destroyed, blanks those slots, and points them at the new group after the rebuild. ``torch.distributed``
is left untouched, and a holder needs no code of its own. Tuples cannot be re-pointed: keep groups out of long-lived
tuples (per-micro-batch tuples are rebuilt anyway).

While released, the blanked slots hold ``RELEASED``, a sentinel that ``torch.distributed`` rejects, so a collective issued
by mistake fails loudly instead of silently running on the world group (which is what ``group=None`` would mean).
"""
from __future__ import annotations

import gc
from typing import Optional

import torch
import torch.distributed as dist


def _torch_internal_holders() -> set:
    """ids of the containers in which ``torch.distributed`` itself tracks groups."""
    from torch.distributed import distributed_c10d as c10d

    w = c10d._world
    out = set()
    for name in ("pg_map", "pg_names", "pg_group_ranks", "pg_backend_config", "pg_to_tag", "tags_to_pg", "pg_coalesce_state"):
        d = getattr(w, name, None)
        if isinstance(d, dict):
            out.add(id(d))
            out.update(id(v) for v in d.values() if isinstance(v, (list, dict)))
    return out


class _Released:
    def __repr__(self) -> str:
        return "<process group released: call reload() first>"


RELEASED = _Released()


class ReloadableGroups:
    def __init__(self):
        self.records: list = []  # creation order: {"ranks", "backend", "timeout", "group", "slots"}
        self.released = False

    # ------------------------------------------------------------------ creation
    def new_group(self, ranks, timeout=None, backend: Optional[str] = None):
        """``dist.new_group`` that remembers how to build the group again. Collective over the world, like the original."""
        assert not self.released, "reload() the groups before creating new ones"
        kw = {}
        if timeout is not None:
            kw["timeout"] = timeout
        if backend is not None:
            kw["backend"] = backend
        g = dist.new_group(list(ranks), **kw)
        self.records.append({"ranks": list(ranks), "backend": backend, "timeout": timeout, "group": g, "slots": []})
        return g

    def _eligible(self, rec: dict, include_host_groups: bool) -> bool:
        """The same answer on every rank, member of the group or not (re-creating a group is collective over the world)."""
        if len(rec["ranks"]) < 2:
            return False
        backend = rec["backend"] or dist.get_backend()
        return include_host_groups or "nccl" in str(backend).lower()  # host-side (gloo) groups pin no device memory

    # ------------------------------------------------------------------ release / reload
    def release(self, include_host_groups: bool = False) -> int:
        """Destroy the groups (newest first). Every rank of the job calls this at the same point, with no collective in
        flight. Returns the device bytes that became free (0 on a CPU job)."""
        if self.released:
            return 0
        cuda = torch.cuda.is_available()
        if cuda:
            torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0] if cuda else 0
        me = dist.get_rank()
        for rec in reversed(self.records):
            rec["slots"], rec["down"] = [], False
            if not self._eligible(rec, include_host_groups):
                continue
            rec["down"] = True
            if me not in rec["ranks"]:
                continue  # nothing of this group lives here; reload() still takes part in creating it again
            g = rec["group"]
            internal = _torch_internal_holders()
            for holder in gc.get_referrers(g):
                if holder is rec or id(holder) in internal:
                    continue  # torch's own tables are cleaned up by destroy_process_group itself
                if isinstance(holder, dict):
                    for k, v in list(holder.items()):
                        if v is g:
                            holder[k] = RELEASED
                            rec["slots"].append((holder, k))
                elif isinstance(holder, list):
                    for k, v in enumerate(holder):
                        if v is g:
                            holder[k] = RELEASED
                            rec["slots"].append((holder, k))
                elif hasattr(holder, "__dict__") and not isinstance(holder, (type, type(gc))):
                    # an instance whose attributes live inline (no separate dict object for the collector to report)
                    d = vars(holder)
                    for k, v in list(d.items()):
                        if v is g:
                            d[k] = RELEASED
                            rec["slots"].append((d, k))
            rec["group"] = RELEASED
            dist.destroy_process_group(g)
            del g
        self.released = True
        if cuda:
            torch.cuda.empty_cache()
            return max(torch.cuda.mem_get_info()[0] - before, 0)
        return 0

    def reload(self) -> int:
        """Create the released groups again, in their original order, and put them back where the old ones were held.
        Returns how many groups this rank got back."""
        if not self.released:
            return 0
        n = 0
        for rec in self.records:
            if not rec.get("down"):
                continue
            kw = {}
            if rec["timeout"] is not None:
                kw["timeout"] = rec["timeout"]
            if rec["backend"] is not None:
                kw["backend"] = rec["backend"]
            g = dist.new_group(rec["ranks"], **kw)  # every rank calls this, member or not
            rec["down"] = False
            if rec["group"] is RELEASED:
                rec["group"] = g
                for holder, k in rec["slots"]:
                    holder[k] = g
                rec["slots"] = []
                n += 1
        self.released = False
        return n


_REGISTRY: Optional[ReloadableGroups] = None


def registry() -> ReloadableGroups:
    global _REGISTRY
    if _REGISTRY is None:
        _REGISTRY = ReloadableGroups()
    return _REGISTRY


def reset_registry() -> None:
    global _REGISTRY
    _REGISTRY = None
