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


def test_prefix_cache_writes_evicted_chains_behind_and_restores_them():
    from cuteafd_b200.engine.kv import PagePool
    from cuteafd_b200.serving.prefix import PrefixCache
    eng = StubCopyEngine(page_bytes=4096)
    hc = HostCache(eng, n_slabs=64, page_bytes=4096, min_tokens=128)
    pool = PagePool(12)
    pc = PrefixCache(pool, max_entries=4, min_tokens=64, max_cached_pages=8, host=hc)
    a = _toks(1, 4) + [7, 8, 9]
    adm = pc.admit(a, reserve_new=1)
    assert adm.hit_tokens == 0
    for i, p in enumerate(adm.seq.pages[:4]):
        eng.device[p] = ("a", i)                                   # what a prefill would have written
    adm.seq.length = len(a)
    pc.capture(a, adm.seq)
    pc.release(adm.seq)
    assert pc.lookup(a) == 256
    pc.evict(100)                                                  # device tier loses the chain; the host tier keeps it
    assert pc.lookup(a) == 0 and hc.lookup(a) == 4 and pc.stats["host_stored_pages"] == 4
    for p in list(eng.device):
        eng.device[p] = None                                       # device pages get reused by someone else
    adm2 = pc.admit(a, reserve_new=1)
    assert adm2.hit_tokens == 256 and pc.stats["host_hits"] == 1
    assert [eng.device[p] for p in adm2.seq.pages[:4]] == [("a", i) for i in range(4)]
    assert pc.lookup(a) == 256                                     # restored pages are ordinary device entries again
    pc.release(adm2.seq)
    # a prompt sharing two pages restores only those
    pc.evict(100)
    b = a[:128] + _toks(2, 2)
    adm3 = pc.admit(b, reserve_new=1)
    assert adm3.hit_tokens == 128


def test_prefix_and_host_tiers_keep_their_books_under_random_traffic():
    """Random admissions, captures, releases and evictions over shared prefixes: page references never leak, restored
    content is always the content that was stored, and both tiers stay within their budgets."""
    import random
    from cuteafd_b200.engine.kv import OutOfPages, PagePool
    from cuteafd_b200.serving.prefix import PrefixCache
    rng = random.Random(3)
    eng = StubCopyEngine(page_bytes=1024)
    hc = HostCache(eng, n_slabs=40, page_bytes=1024, min_tokens=64)
    pool = PagePool(48)
    pc = PrefixCache(pool, max_entries=6, min_tokens=64, max_cached_pages=20, host=hc)
    prefixes = [_toks(10 + i, rng.randrange(1, 5)) for i in range(8)]
    content: dict = {}                                          # (prefix id, page index) written by the "prefill"
    live = []
    for step in range(600):
        if live and rng.random() < 0.45:
            adm, toks = live.pop(rng.randrange(len(live)))
            pc.release(adm.seq)
            continue
        pid = rng.randrange(len(prefixes))
        toks = prefixes[pid] + [rng.randrange(5)] * rng.randrange(1, 40)
        try:
            adm = pc.admit(toks, reserve_new=1)
        except OutOfPages:
            continue
        n_full = len(prefixes[pid]) // 64
        for i in range(n_full):
            page = adm.seq.pages[i]
            if i * 64 < adm.hit_tokens:
                assert eng.device.get(page) == (pid, i), "a restored or shared page holds someone else's content"
            else:
                eng.device[page] = (pid, i)                     # computed by this request
        adm.seq.length = len(toks)
        pc.capture(toks, adm.seq)
        live.append((adm, toks))
        if rng.random() < 0.1:
            pc.evict(rng.randrange(1, 8))
        assert pc.n_nodes <= 20 + 8 and len(hc.pages) + len(hc.free) == 40
    for adm, _ in live:
        pc.release(adm.seq)
    pc.evict(10 ** 6)
    assert pool.n_free == 47 and all(r == 0 for r in pool.refs[1:])          # nothing leaked (page 0 is reserved)
    assert hc.stats["restored_pages"] > 0 and pc.stats["host_hits"] > 0


def test_restore_survives_both_tiers_being_full():
    """Device pool of 9 pages, 4 host slabs, three 3-page prompts A, B, C, then A again: making room for A's restore evicts
    device chains, whose write-behind evicts host pages.  The pages being restored are pinned, nothing leaks, no KeyError."""
    from cuteafd_b200.engine.kv import PagePool
    from cuteafd_b200.serving.prefix import PrefixCache
    eng = StubCopyEngine(page_bytes=4096)
    hc = HostCache(eng, n_slabs=4, page_bytes=4096, min_tokens=64)
    pool = PagePool(9)
    pc = PrefixCache(pool, max_entries=8, min_tokens=64, max_cached_pages=9, host=hc)
    prompts = {t: _toks(t, 3) + [1] for t in (1, 2, 3)}
    for t in (1, 2, 3, 1, 2, 3, 1):
        adm = pc.admit(prompts[t], reserve_new=1)
        for i, p in enumerate(adm.seq.pages[:3]):
            if i * 64 >= adm.hit_tokens:
                eng.device[p] = (t, i)
        for i, p in enumerate(adm.seq.pages[:3]):
            assert eng.device[p] == (t, i)                          # restored pages carry this prompt's content
        adm.seq.length = len(prompts[t])
        pc.capture(prompts[t], adm.seq)
        pc.release(adm.seq)
        held = pc.n_nodes
        assert pool.n_free + held == pool.n_pages - pool.reserved   # every page is either free or owned by the tree
    assert all(hp.refs == 0 for hp in hc.pages.values())


def test_restore_stops_at_a_missing_page_and_reports_the_count():
    eng = StubCopyEngine(page_bytes=1000)
    hc = HostCache(eng, n_slabs=8, page_bytes=1000, min_tokens=64)
    a = _toks(1, 4)
    for p in range(4):
        eng.device[p] = ("a", p)
    hc.store(a, [0, 1, 2, 3])
    from cuteafd_b200.serving.hostcache import chain_key
    key = b""
    for d in range(3):
        key = chain_key(key, tuple(a[d * 64:(d + 1) * 64]))
    hc.free.append(hc.pages.pop(key).slab)                          # page 2 disappears
    assert hc.restore(a, 0, [10, 11, 12, 13]) == 2
