"""Host-only C++ runtime (miles_b200._native): page pool, scheduler, quorum store, router table."""
import pytest

from miles_b200.ops import _native


@pytest.fixture(scope="module")
def N():
    return _native.load()


def test_page_pool_all_or_nothing_and_double_free(N):
    p = N.PagePool(6)
    assert p.num_free == 5 and p.alloc(6) is None
    a = p.alloc(3)
    assert sorted(a) == [1, 2, 3] and p.num_free == 2
    p.release(a)
    assert p.num_free == 5
    with pytest.raises(Exception):
        p.release([1])  # already free
    with pytest.raises(Exception):
        p.release([0])  # reserved page


def test_quorum_changes_on_timeout_join_and_evict(N):
    q = N.QuorumStore(timeout_s=10.0)
    q.heartbeat("cell-0", 0.0)
    qid = q.heartbeat("cell-1", 1.0)
    assert q.quorum(5.0) == (qid, ["cell-0", "cell-1"]) and q.rank_of("cell-1") == 1
    qid2, members = q.quorum(10.5)  # cell-0 has not been heard from for more than 10 s
    assert qid2 == qid + 1 and members == ["cell-1"]
    assert q.heartbeat("cell-0", 11.0) == qid2 + 1  # it rejoins: a new quorum
    assert q.evict("cell-1") == qid2 + 2 and q.quorum(11.0)[1] == ["cell-0"] and q.rank_of("cell-1") == -1


def test_router_table_least_inflight_and_quarantine(N):
    r = N.RouterTable(2)
    for u in ("a", "b"):
        r.add(u)
    first, second = r.acquire(), r.acquire()
    assert {first, second} == {"a", "b"}
    r.release("a", True)
    assert r.acquire() == "a"  # fewest in flight
    r.release("b", False)
    r.release("a", False)
    r.report_health("a", False)  # second consecutive failure
    assert r.urls(True) == ["b"] and r.acquire() == "b"
    r.readmit("a")
    assert sorted(r.urls(True)) == ["a", "b"]
    assert r.remove("b") and r.urls(False) == ["a"]
