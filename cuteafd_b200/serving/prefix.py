"""Exact prefix cache over the paged KV store (device tier).

Sequences are cut into 64-token pages; a radix tree keyed by page-sized token blocks maps a prompt prefix to the
refcounted KV pages that hold it.  `admit` forks those pages into a new sequence (no copy, no recompute); the
restored state is byte-identical to what a cold prefill would have produced because the pages ARE the ones a
prefill wrote.  Snapshots are taken at page boundaries (`capture`), a cancelled prefill is parked as a snapshot,
least-recently-used entries are evicted when the entry or page budget is exceeded, and a partial last page is never
shared (the tail is recomputed), which keeps sharing exact without copy-on-write.

Reference: cuteafd-engine/src/prefix/cache.rs:315-888 (admit / capture / park / release / tick),
prefix/points.rs:55 (snapshot points), cuteafd-core/src/prefix.rs:1-57 (radix + reuse rule).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field

from ..engine.kv import PAGE, OutOfPages, PagePool, SeqKV


@dataclass
class Node:
    page: int = -1                      # KV page holding this block (-1 for the root)
    children: dict = field(default_factory=dict)
    parent: "Node | None" = None
    key: tuple = ()
    last_used: int = 0
    kind: str = "prompt"                # prompt | turn | parked
    logits_row: object = None           # retained last-row logits for whole-prompt hits
    hkey: bytes | None = None           # content identity of the chain up to this page (host tier key), computed on demand


@dataclass
class Admission:
    seq: SeqKV
    hit_tokens: int                     # tokens restored from the cache (multiple of PAGE)
    logits_row: object = None           # set when the whole prompt was cached (minus nothing to compute)


class PrefixCache:
    def __init__(self, pool: PagePool, max_entries: int = 20, min_tokens: int = 64, max_cached_pages: int | None = None, host=None):
        """`host` is an optional `HostCache`: evicted chains are written behind into it and a prompt whose prefix lives only
        there gets its pages copied back into fresh device pages on admission (cuteafd-hostcache/src/lib.rs:1-24)."""
        self.pool, self.max_entries, self.min_tokens = pool, max_entries, min_tokens
        self.host = host
        self.max_cached_pages = max_cached_pages if max_cached_pages is not None else pool.n_pages // 2
        self.root = Node()
        self.clock = itertools.count(1)
        self.n_nodes = 0
        self.stats = {"lookups": 0, "hits": 0, "hit_tokens": 0, "captures": 0, "evictions": 0, "parked": 0, "deferred": 0,
                      "host_hits": 0, "host_hit_tokens": 0, "host_stored_pages": 0}

    # ------------------------------------------------------------------ lookup / admit
    def _walk(self, tokens: list[int]):
        node, depth = self.root, 0
        while (depth + 1) * PAGE <= len(tokens):
            key = tuple(tokens[depth * PAGE:(depth + 1) * PAGE])
            nxt = node.children.get(key)
            if nxt is None:
                break
            node, depth = nxt, depth + 1
        return node, depth

    def lookup(self, tokens: list[int]) -> int:
        """Number of prompt tokens a new request could restore."""
        return self._walk(tokens)[1] * PAGE

    def admit(self, tokens: list[int], reserve_new: int = 1) -> Admission:
        """New sequence for `tokens`: cached full pages are shared, pages for the rest are allocated.
        At least one prompt token is always left to compute so the request gets fresh last-row logits, unless
        the cached node kept them.  Raises OutOfPages (after trying eviction) when the pool cannot hold it."""
        self.stats["lookups"] += 1
        node, depth = self._walk(tokens)
        if self.host is not None:
            node, depth = self._extend_from_host(tokens, node, depth)
        logits_row = None
        if depth * PAGE == len(tokens):
            if node.logits_row is not None:
                logits_row = node.logits_row
            else:
                node, depth = node.parent, depth - 1       # recompute the last page to get logits
        if depth * PAGE < self.min_tokens:
            node, depth, logits_row = self.root, 0, None
        pages, n = [], node
        while n is not self.root:
            pages.append(n.page)
            n.last_used = next(self.clock)
            n = n.parent
        pages.reverse()
        seq = SeqKV(pages=list(pages), length=depth * PAGE)
        need = seq.pages_needed(len(tokens) + reserve_new)
        if not self.pool.can_alloc(need):
            self.evict(need - self.pool.n_free, protect=set(pages))
        if not self.pool.can_alloc(need):
            self.stats["deferred"] += 1
            raise OutOfPages(f"need {need} pages, {self.pool.n_free} free")
        for p in pages:
            self.pool.retain(p)
        seq.ensure(self.pool, len(tokens) + reserve_new)
        if depth:
            self.stats["hits"] += 1
            self.stats["hit_tokens"] += depth * PAGE
        return Admission(seq, depth * PAGE, logits_row)

    # ------------------------------------------------------------------ host tier
    def _chain(self, n: Node):
        """Nodes from the first page to `n`."""
        out = []
        while n is not self.root:
            out.append(n)
            n = n.parent
        out.reverse()
        return out

    def _hkeys(self, chain) -> list:
        from .hostcache import chain_key
        prev = b""
        for n in chain:
            if n.hkey is None:
                n.hkey = chain_key(prev, n.key)
            prev = n.hkey
        return [n.hkey for n in chain]

    def _extend_from_host(self, tokens: list[int], node: Node, depth: int):
        """Pages [depth, n_host) of the prompt exist only on the host: copy them into fresh device pages and hang them
        into the tree, so the admission below (and later requests) see an ordinary device hit."""
        n_host = self.host.lookup(tokens)
        if n_host <= depth or n_host * PAGE < self.min_tokens:
            return node, depth
        chain_pages = {n.page for n in self._chain(node)}
        want = n_host - depth
        # Making room on the device evicts chains, whose write-behind may in turn evict host pages: hold the pages of THIS
        # prefix on the host until they have been copied back.
        self.host.pin(tokens, n_host, +1)
        pages = []
        try:
            if not self.pool.can_alloc(want):
                self.evict(want - self.pool.n_free, protect=chain_pages)
            want = min(want, self.pool.n_free)
            if want <= 0:
                return node, depth
            pages = [self.pool.alloc() for _ in range(want)]        # the tree owns these references
            got = self.host.restore(tokens, depth, pages)
        except Exception:
            for p in pages:
                self.pool.release(p)
            raise
        finally:
            self.host.pin(tokens, n_host, -1)
        for p in pages[got:]:                                       # pages the host no longer held: back to the pool
            self.pool.release(p)
        pages, want = pages[:got], got
        if not pages:
            return node, depth
        for i, page in enumerate(pages):
            key = tuple(tokens[(depth + i) * PAGE:(depth + i + 1) * PAGE])
            nxt = Node(page=page, parent=node, key=key, kind="host")
            nxt.last_used = next(self.clock)
            node.children[key] = nxt
            self.n_nodes += 1
            node = nxt
        self.stats["host_hits"] += 1
        self.stats["host_hit_tokens"] += want * PAGE
        return node, depth + want

    # ------------------------------------------------------------------ capture / park
    def capture(self, tokens: list[int], seq: SeqKV, kind: str = "prompt", logits_row=None) -> int:
        """Record the full pages of `seq` that hold `tokens[:seq.length]`.  Returns tokens now cached."""
        n_full = min(len(tokens), seq.length) // PAGE
        node = self.root
        for d in range(n_full):
            key = tuple(tokens[d * PAGE:(d + 1) * PAGE])
            nxt = node.children.get(key)
            if nxt is None:
                nxt = Node(page=seq.pages[d], parent=node, key=key, kind=kind)
                self.pool.retain(seq.pages[d])
                node.children[key] = nxt
                self.n_nodes += 1
            nxt.last_used = next(self.clock)
            node = nxt
        if logits_row is not None and n_full * PAGE == len(tokens) and node is not self.root:
            node.logits_row = logits_row
        self.stats["captures"] += 1
        self._trim()
        return n_full * PAGE

    def park(self, tokens: list[int], seq: SeqKV) -> int:
        """A cancelled prefill keeps what it computed as a snapshot instead of throwing it away."""
        self.stats["parked"] += 1
        return self.capture(tokens[:seq.length], seq, kind="parked")

    def release(self, seq: SeqKV):
        seq.release(self.pool)

    # ------------------------------------------------------------------ eviction
    def _leaves(self):
        out, stack = [], [self.root]
        while stack:
            n = stack.pop()
            if n is not self.root and not n.children:
                out.append(n)
            stack.extend(n.children.values())
        return out

    def _drop(self, n: Node):
        if self.host is not None:
            chain = self._chain(n)
            self.stats["host_stored_pages"] += self.host.store([], [c.page for c in chain], keys=self._hkeys(chain))
        del n.parent.children[n.key]
        self.pool.release(n.page)
        self.n_nodes -= 1
        self.stats["evictions"] += 1

    def evict(self, n_pages: int, protect: set | None = None) -> int:
        """Drop least-recently-used leaves until `n_pages` pages came back to the pool (or nothing is left)."""
        freed, protect = 0, protect or set()
        while freed < n_pages:
            leaves = [l for l in self._leaves() if l.page not in protect]
            if not leaves:
                break
            victim = min(leaves, key=lambda l: l.last_used)
            before = self.pool.n_free
            self._drop(victim)
            freed += self.pool.n_free - before
            if self.pool.n_free == before and not [l for l in self._leaves() if l.page not in protect]:
                break
        return freed

    def _entries(self) -> int:
        return len(self._leaves())

    def _trim(self):
        while self._entries() > self.max_entries or self.n_nodes > self.max_cached_pages:
            leaves = self._leaves()
            if not leaves:
                break
            self._drop(min(leaves, key=lambda l: l.last_used))

    def tick(self):
        self._trim()

    def snapshot(self) -> dict:
        return dict(self.stats, entries=self._entries(), cached_pages=self.n_nodes, free_pages=self.pool.n_free)
