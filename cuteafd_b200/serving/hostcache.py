"""Pinned host-memory tier behind the device prefix cache.

When the device tier evicts a snapshot its pages are written behind into a pool of fixed-size pinned slabs instead
of being lost; a later request whose prefix lives only on the host gets its pages copied back (host-to-device) in
milliseconds instead of recomputing them.  Pages are shared exactly: identical content (same token-block chain)
is stored once and refcounted.  Budgets bound total bytes and keep headroom; least-recently-used chains are
dropped first.  All copies go through a `CopyEngine` so the whole tier runs against `StubCopyEngine` and a virtual
clock in tests - the reference ships the same split (cuteafd-hostcache/src/copy.rs:36,190; sim.rs).

Reference: cuteafd-hostcache/src/lib.rs:1-24 (write-behind tier, exact page sharing, budgets), cache.rs, pool.rs.
"""
from __future__ import annotations

import hashlib
import itertools
from dataclasses import dataclass, field


class CopyEngine:
    """Moves KV pages between the device pool and host slabs."""
    def d2h(self, device_page: int, slab: int): ...
    def h2d(self, slab: int, device_page: int): ...
    def synchronize(self): ...

    def d2h_many(self, pairs: list):
        """`pairs` = [(device page, slab), ...]; engines that can batch override this."""
        for page, slab in pairs:
            self.d2h(page, slab)

    def h2d_many(self, pairs: list):
        for page, slab in pairs:
            self.h2d(slab, page)


class StubCopyEngine(CopyEngine):
    """Records copies and charges virtual time (bytes / bandwidth + latency)."""

    def __init__(self, page_bytes: int, gbps: float = 50.0, latency_us: float = 10.0):
        self.page_bytes, self.gbps, self.latency_us = page_bytes, gbps, latency_us
        self.clock_us = 0.0
        self.log: list = []
        self.device: dict = {}      # device page -> content tag
        self.host: dict = {}        # slab -> content tag

    def _charge(self):
        self.clock_us += self.latency_us + self.page_bytes / (self.gbps * 1e3)

    def d2h(self, device_page, slab):
        self.host[slab] = self.device.get(device_page)
        self.log.append(("d2h", device_page, slab))
        self._charge()

    def h2d(self, slab, device_page):
        self.device[device_page] = self.host.get(slab)
        self.log.append(("h2d", slab, device_page))
        self._charge()

    def synchronize(self):
        pass


class CudaCopyEngine(CopyEngine):
    """Copies pages of the engine's KV tensor [layers, slots, ...] to/from one pinned host tensor on a side stream.

    A batch of pages moves in ONE kernel launch that reads or writes the pinned slabs through their device mapping
    (`ops.kv_pages_copy`).  Ordering against the compute stream is by stream dependencies only, never a host wait: the
    side stream first waits for the work already queued on the caller's stream (the pages' content is final; a page about
    to be overwritten is no longer read), and the caller's stream then waits for the copy (a page released after a
    write-behind is not reused before it has left; a restored page is complete before attention reads it)."""

    def __init__(self, kv, n_slabs: int, page_tokens: int = 64):
        import torch
        self.kv, self.page_tokens = kv, page_tokens
        L = kv.shape[0]
        self.host = torch.empty((n_slabs, L, page_tokens) + tuple(kv.shape[2:]), dtype=kv.dtype).pin_memory()
        self.stream = torch.cuda.Stream(device=kv.device)
        self.page_bytes = self.host[0].numel() * self.host.element_size()
        self.launches = 0

    def _move(self, pairs, to_pool: bool):
        import torch
        from .. import ops
        if not pairs:
            return
        cur = torch.cuda.current_stream(self.kv.device)
        t = torch.tensor(pairs, dtype=torch.int32).pin_memory().to(self.kv.device, non_blocking=True)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            ops.kv_pages_copy(self.kv, t, self.host, to_pool)
        t.record_stream(self.stream)
        cur.wait_stream(self.stream)
        self.launches += 1

    def d2h_many(self, pairs):
        self._move(pairs, True)

    def h2d_many(self, pairs):
        self._move(pairs, False)

    def d2h(self, device_page, slab):
        self._move([(device_page, slab)], True)

    def h2d(self, slab, device_page):
        self._move([(device_page, slab)], False)

    def synchronize(self):
        self.stream.synchronize()


@dataclass
class HostPage:
    slab: int
    refs: int = 0
    last_used: int = 0


def chain_key(parent_key: bytes, block: tuple) -> bytes:
    """Content identity of a page = hash of (identity of the prefix before it, its 64 tokens)."""
    h = hashlib.blake2b(digest_size=16)
    h.update(parent_key)
    h.update(repr(block).encode())
    return h.digest()


class HostCache:
    def __init__(self, copy: CopyEngine, n_slabs: int, page_bytes: int, budget_bytes: int | None = None, headroom_bytes: int = 0,
                 min_tokens: int = 512, page_tokens: int = 64):
        self.copy, self.page_bytes, self.page_tokens, self.min_tokens = copy, page_bytes, page_tokens, min_tokens
        usable = n_slabs if budget_bytes is None else min(n_slabs, max(0, (budget_bytes - headroom_bytes)) // page_bytes)
        self.free = list(range(usable - 1, -1, -1))
        self.pages: dict[bytes, HostPage] = {}
        self.clock = itertools.count(1)
        self.stats = {"stored_pages": 0, "shared_hits": 0, "restored_pages": 0, "evicted_pages": 0, "rejected": 0, "lookups": 0, "hits": 0}

    # ---- write-behind on device eviction
    def store(self, tokens: list[int], device_pages: list[int], keys: list | None = None) -> int:
        """Persist the pages of a prefix (tokens cover len(device_pages) full pages).  Returns pages newly written.
        `keys` may carry the chain keys of the pages when the caller keeps them (saves re-hashing the tokens)."""
        n = len(device_pages)
        if n * self.page_tokens < self.min_tokens:
            self.stats["rejected"] += 1
            return 0
        key, written, batch = b"", 0, []
        for d in range(n):
            key = keys[d] if keys is not None else chain_key(key, tuple(tokens[d * self.page_tokens:(d + 1) * self.page_tokens]))
            hp = self.pages.get(key)
            if hp is None:
                if not self.free and not self._evict_one(protect=key):
                    break
                if not self.free:
                    break
                hp = HostPage(self.free.pop())
                batch.append((device_pages[d], hp.slab))
                self.pages[key] = hp
                self.stats["stored_pages"] += 1
                written += 1
            else:
                self.stats["shared_hits"] += 1
            hp.last_used = next(self.clock)
        self.copy.d2h_many(batch)
        return written

    # ---- restore
    def lookup(self, tokens: list[int]) -> int:
        """How many leading full pages of `tokens` the host tier holds."""
        self.stats["lookups"] += 1
        key, n = b"", 0
        while (n + 1) * self.page_tokens <= len(tokens):
            key = chain_key(key, tuple(tokens[n * self.page_tokens:(n + 1) * self.page_tokens]))
            if key not in self.pages:
                break
            n += 1
        return n

    def pin(self, tokens: list[int], n_pages: int, delta: int = 1) -> None:
        """Hold (`delta` = 1) or let go of (`delta` = -1) the first `n_pages` host pages of a prefix: pinned pages are never
        chosen by `_evict_one`, so a restore that must first make room on the device (whose evictions write behind into this
        tier) cannot lose the pages it is about to copy back."""
        key = b""
        for d in range(n_pages):
            key = chain_key(key, tuple(tokens[d * self.page_tokens:(d + 1) * self.page_tokens]))
            hp = self.pages.get(key)
            if hp is None:
                break
            hp.refs = max(0, hp.refs + delta)

    def restore(self, tokens: list[int], first_page: int, device_pages: list[int]) -> int:
        """Copy host pages [first_page, first_page + len(device_pages)) of the prefix into the given device pages.  Stops at the
        first page the tier no longer holds and returns how many pages were restored (the caller releases the rest)."""
        key, batch = b"", []
        for d in range(first_page + len(device_pages)):
            key = chain_key(key, tuple(tokens[d * self.page_tokens:(d + 1) * self.page_tokens]))
            hp = self.pages.get(key)
            if hp is None:
                break
            if d >= first_page:
                hp.last_used = next(self.clock)
                batch.append((device_pages[d - first_page], hp.slab))
                self.stats["restored_pages"] += 1
        self.copy.h2d_many(batch)
        self.copy.synchronize()
        if batch:
            self.stats["hits"] += 1
        return len(batch)

    def _evict_one(self, protect: bytes | None = None) -> bool:
        cands = [(hp.last_used, k) for k, hp in self.pages.items() if hp.refs == 0 and k != protect]
        if not cands:
            return False
        _, k = min(cands)
        self.free.append(self.pages.pop(k).slab)
        self.stats["evicted_pages"] += 1
        return True

    def snapshot(self) -> dict:
        return dict(self.stats, resident_pages=len(self.pages), free_slabs=len(self.free), bytes=len(self.pages) * self.page_bytes)


def attach_host_tier(engine, gib: float, min_tokens: int = 512, page_tokens: int = 64) -> "HostCache":
    """Host tier of `gib` GiB of pinned memory behind an engine's paged KV store (any engine exposing `kv` as
    [layers, slots, ...]); pass the result to `PrefixCache(..., host=...)`."""
    copy_probe = engine.kv[0, :page_tokens]
    page_bytes = engine.kv.shape[0] * copy_probe.numel() * copy_probe.element_size()
    n_slabs = max(1, int(gib * (1 << 30)) // page_bytes)
    copy = CudaCopyEngine(engine.kv, n_slabs, page_tokens)
    return HostCache(copy, n_slabs, page_bytes, min_tokens=min_tokens, page_tokens=page_tokens)


def simulate(n_requests: int = 200, n_prefixes: int = 12, prefix_pages: int = 40, device_pages: int = 128, host_slabs: int = 512,
             page_bytes: int = 91136, seed: int = 0) -> dict:
    """Virtual-clock simulation of device tier + host tier under a skewed prefix workload: returns hit counts and the
    time saved versus recomputing (reference: cuteafd-hostcache/src/sim.rs)."""
    import random
    rnd = random.Random(seed)
    eng = StubCopyEngine(page_bytes)
    host = HostCache(eng, host_slabs, page_bytes, min_tokens=64)
    resident: dict[int, int] = {}          # prefix id -> lru stamp on the device tier
    capacity = device_pages // prefix_pages
    stamp = itertools.count(1)
    recompute_us_per_page = 64 * 120.0      # ~120 us per prefill token
    saved = cold = dev_hits = host_hits = 0
    for _ in range(n_requests):
        pid = min(int(rnd.expovariate(0.35)), n_prefixes - 1)
        toks = [pid * 1000 + (i // 64) for i in range(prefix_pages * 64)]
        if pid in resident:
            dev_hits += 1
            saved += prefix_pages * recompute_us_per_page
        else:
            n = host.lookup(toks)
            if n:
                host_hits += 1
                t0 = eng.clock_us
                host.restore(toks, 0, list(range(n)))
                saved += n * recompute_us_per_page - (eng.clock_us - t0)
            else:
                cold += 1
            if len(resident) >= capacity:
                victim = min(resident, key=resident.get)
                vt = [victim * 1000 + (i // 64) for i in range(prefix_pages * 64)]
                for p in range(prefix_pages):
                    eng.device[p] = (victim, p)
                host.store(vt, list(range(prefix_pages)))
                del resident[victim]
        resident[pid] = next(stamp)
    return {"device_hits": dev_hits, "host_hits": host_hits, "cold": cold, "saved_ms": saved / 1e3, "copy_ms": eng.clock_us / 1e3,
            "host": host.snapshot()}
