"""Prefix (radix) cache over KV pages.

Requests whose token sequences start alike share the KV pages of the common start instead of recomputing them: the
eight samples of one GRPO prompt, the turns of a multi-turn / agentic conversation (every turn re-sends the whole
conversation), evaluation prompts with a shared system prompt. The tree is page granular: a node stands for one *full*
page (``page_size`` tokens) and is keyed by those tokens under its parent, so a lookup walks whole pages and a cached
page is immutable (new tokens always go to pages the request owns alone).

Ownership: a page in the tree belongs to the cache. Requests that use it hold a reference on its node (``lock``);
nodes without references stay cached until the pool runs dry, then least-recently-used leaves are evicted and their
pages returned (``evict``). A weight update invalidates everything (``clear``): cached keys / values were computed with
the old weights.

A node may carry a payload per page (the routed experts of its tokens, which routing replay needs for cached prompt
tokens as well); ``match(..., need_payload=True)`` stops at the first node without one.

Reference behaviour: SGLang's radix cache, on by default in the engines the reference launches
(miles/backends/sglang_utils/sglang_engine.py; ``--sglang-disable-radix-cache`` turns it off) and the
``cached_tokens`` / prefix-cache hit-rate metrics of miles/rollout/generate_utils/generate_endpoint_utils.py.
"""
from __future__ import annotations

import itertools
from typing import Optional, Sequence


class _Node:
    __slots__ = ("key", "page", "parent", "children", "refs", "tick", "payload", "orphan")

    def __init__(self, key, page, parent):
        self.key, self.page, self.parent = key, page, parent
        self.children: dict = {}
        self.refs = 0
        self.tick = 0
        self.payload = None
        self.orphan = False   # detached by clear() while still referenced: its page goes back when the last user lets go


class PrefixCache:
    def __init__(self, page_size: int):
        self.page_size = int(page_size)
        self.root = _Node(None, -1, None)
        self._clock = itertools.count(1)
        self.epoch = 0         # bumped by clear(): sequences computed before it are not offered to the cache afterwards
        self.num_pages = 0
        self.hits = 0          # tokens served from the cache
        self.queries = 0       # tokens asked for

    # ------------------------------------------------------------------ lookup
    def match(self, tokens: Sequence[int], max_tokens: Optional[int] = None, need_payload: bool = False) -> list:
        """The nodes of the longest cached prefix of ``tokens`` made of full pages, at most ``max_tokens`` tokens long
        (a prefill must keep at least one token to compute, so callers pass ``len(tokens) - 1``)."""
        ps = self.page_size
        limit = len(tokens) if max_tokens is None else min(len(tokens), max_tokens)
        node, out = self.root, []
        tick = next(self._clock)
        for p in range(limit // ps):
            child = node.children.get(tuple(tokens[p * ps:(p + 1) * ps]))
            if child is None or (need_payload and child.payload is None):
                break
            child.tick = tick
            out.append(child)
            node = child
        self.queries += len(tokens)
        self.hits += len(out) * ps
        return out

    @staticmethod
    def lock(nodes: Sequence[_Node]) -> None:
        for n in nodes:
            n.refs += 1

    @staticmethod
    def unlock(nodes: Sequence[_Node]) -> list:
        """Drop one reference per node. Returns the pages of nodes that ``clear`` had detached and that nobody uses any
        more (the caller hands them back to the pool)."""
        free = []
        for n in nodes:
            assert n.refs > 0
            n.refs -= 1
            if n.orphan and n.refs == 0:
                free.append(n.page)
        return free

    # ------------------------------------------------------------------ insertion
    def insert(self, tokens: Sequence[int], pages: Sequence[int], payloads: Optional[Sequence] = None, skip: int = 0,
               stop_at_duplicate: bool = False) -> tuple:
        """Offer the full pages of a computed sequence. ``pages[i]`` holds tokens ``[i*ps, (i+1)*ps)``; the first
        ``skip`` pages are already tree pages (they came from ``match``). Returns ``(nodes, duplicates)``: the node of
        every full page in order (existing or new; the caller should hold / take references on them instead of owning
        the pages) and the offered pages that were *not* taken because an equal page was cached already (the caller
        releases those). ``stop_at_duplicate``: end at the first such page instead (the returned nodes then cover only
        the pages before it)."""
        ps = self.page_size
        node, nodes, dup = self.root, [], []
        tick = next(self._clock)
        for i in range(min(len(tokens) // ps, len(pages))):
            key = tuple(tokens[i * ps:(i + 1) * ps])
            child = node.children.get(key)
            if child is None:
                assert i >= skip, "a page that came from the cache must still be in it"
                child = _Node(key, int(pages[i]), node)
                node.children[key] = child
                self.num_pages += 1
            elif i >= skip and child.page != int(pages[i]):
                if stop_at_duplicate:   # a request in flight keeps using its own copy: its later pages stay its own too
                    break
                dup.append(int(pages[i]))
            if payloads is not None and child.payload is None and i < len(payloads):
                child.payload = payloads[i]
            child.tick = tick
            nodes.append(child)
            node = child
        return nodes, dup

    # ------------------------------------------------------------------ eviction
    def evict(self, want_pages: int) -> list:
        """Free up to ``want_pages`` pages: least recently used leaves that nobody references. Returns the page ids."""
        freed = []
        while len(freed) < want_pages:
            leaves = [n for n in self._leaves() if n.refs == 0]
            if not leaves:
                break
            leaves.sort(key=lambda n: n.tick)
            for n in leaves:
                if len(freed) >= want_pages:
                    break
                del n.parent.children[n.key]
                self.num_pages -= 1
                freed.append(n.page)
        return freed

    def _leaves(self):
        stack = [self.root]
        while stack:
            n = stack.pop()
            if not n.children and n is not self.root:
                yield n
            stack.extend(n.children.values())

    def clear(self) -> list:
        """Forget everything (weights changed). Returns the pages of nodes nobody references; referenced pages stay
        with the requests that hold them (their nodes are detached, so they are never matched again)."""
        free = []
        stack = list(self.root.children.values())
        while stack:
            n = stack.pop()
            stack.extend(n.children.values())
            if n.refs == 0:
                free.append(n.page)
            else:
                n.orphan = True
            n.children = {}
            n.parent = None
        self.root = _Node(None, -1, None)
        self.num_pages = 0
        self.epoch += 1
        return free

    def hit_rate(self) -> float:
        return self.hits / self.queries if self.queries else 0.0
