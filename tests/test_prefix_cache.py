"""The page-granular prefix tree of the engine: matching, reference counts, eviction order, invalidation."""
from miles_b200.engine.prefix_cache import PrefixCache


def seq(*blocks):
    out = []
    for b in blocks:
        out += [b * 10 + j for j in range(4)]
    return out


def test_match_insert_and_duplicates():
    c = PrefixCache(page_size=4)
    a = seq(1, 2, 3) + [7]                      # three full pages and a partial one
    assert c.match(a, len(a) - 1) == []
    nodes, dup = c.insert(a, [11, 12, 13, 14])
    assert [n.page for n in nodes] == [11, 12, 13] and dup == [] and c.num_pages == 3
    # a second sequence with the same two first pages, computed independently into its own pages
    b = seq(1, 2, 9)
    hit = c.match(b, len(b) - 1)
    assert [n.page for n in hit] == [11, 12]
    nodes, dup = c.insert(b, [21, 22, 23])      # offered without using the hit: its first two pages are duplicates
    assert [n.page for n in nodes] == [11, 12, 23] and dup == [21, 22] and c.num_pages == 4
    # at least one token is left to compute: a fully cached sequence matches one page less
    assert len(c.match(seq(1, 2, 3), len(seq(1, 2, 3)) - 1)) == 2
    assert c.hit_rate() > 0


def test_eviction_is_lru_over_unreferenced_leaves():
    c = PrefixCache(page_size=4)
    na, _ = c.insert(seq(1, 2), [1, 2])
    nb, _ = c.insert(seq(1, 3), [1, 3], skip=1)
    nc, _ = c.insert(seq(4), [4])
    c.lock(nb)                                   # a running request uses 1 -> 3
    c.match(seq(4, 0), 4)                        # touch 4: now the least recently used free leaf is page 2
    assert c.evict(1) == [2]
    assert c.evict(5) == [4]                     # page 3 and its parent are referenced: they stay
    assert c.num_pages == 2
    assert c.unlock(nb) == []
    assert sorted(c.evict(5)) == [1, 3] and c.num_pages == 0


def test_payload_requirement_and_clear():
    c = PrefixCache(page_size=4)
    c.insert(seq(1, 2), [1, 2], payloads=["r1"])           # only the first page carries routed experts
    assert len(c.match(seq(1, 2, 3), 11)) == 2
    assert len(c.match(seq(1, 2, 3), 11, need_payload=True)) == 1
    held = c.match(seq(1, 2, 3), 11)
    c.lock(held[:1])
    e0 = c.epoch
    assert c.clear() == [2]                      # page 1 is still in use: it stays with its user
    assert c.epoch == e0 + 1 and c.match(seq(1, 2), 7) == [] and c.num_pages == 0
    assert c.unlock(held[:1]) == [1]             # ... and goes back to the pool when the user lets go
