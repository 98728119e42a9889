"""Host tier of the prefix cache against the stub copy engine and the virtual-clock simulator (CPU only)."""
from cuteafd_b200.serving.hostcache import HostCache, StubCopyEngine, simulate


def _toks(tag, pages):
    return [tag * 100000 + i for i in range(pages * 64)]


def test_store_restore_is_exact_and_shares_identical_pages():
    eng = StubCopyEngine(page_bytes=1 << 16)
    hc = HostCache(eng, n_slabs=16, page_bytes=1 << 16, min_tokens=128)
    a = _toks(1, 4)
    for p in range(4):
        eng.device[10 + p] = ("a", p)
    assert hc.store(a, [10, 11, 12, 13]) == 4
    # a second snapshot sharing the first three pages stores only its new page
    b = a[:3 * 64] + _toks(2, 1)
    eng.device[20] = ("b", 3)
    assert hc.store(b, [10, 11, 12, 20]) == 1 and hc.stats["shared_hits"] == 3
    assert hc.lookup(a) == 4 and hc.lookup(b) == 4 and hc.lookup(_toks(3, 2)) == 0
    hc.restore(b, 1, [40, 41, 42])
    assert [eng.device[p] for p in (40, 41, 42)] == [("a", 1), ("a", 2), ("b", 3)]       # byte-identical content came back
    assert hc.store(_toks(5, 1), [1]) == 0 and hc.stats["rejected"] == 1                 # below min_tokens


def test_budget_and_lru_eviction():
    eng = StubCopyEngine(page_bytes=1000)
    hc = HostCache(eng, n_slabs=100, page_bytes=1000, budget_bytes=9000, headroom_bytes=3000, min_tokens=64)
    assert hc.snapshot()["free_slabs"] == 6
    hc.store(_toks(1, 3), [0, 1, 2])
    hc.store(_toks(2, 3), [3, 4, 5])
    hc.lookup(_toks(1, 3)), hc.restore(_toks(1, 3), 0, [7, 8, 9])      # touch chain 1 so chain 2 is the LRU
    hc.store(_toks(3, 2), [0, 1])
    assert hc.stats["evicted_pages"] == 2 and hc.lookup(_toks(1, 3)) == 3 and hc.lookup(_toks(2, 3)) < 3


def test_simulator_shows_the_host_tier_paying_off():
    r = simulate(n_requests=300)
    assert r["host_hits"] > 0 and r["saved_ms"] > r["copy_ms"] and r["device_hits"] + r["host_hits"] + r["cold"] == 300
