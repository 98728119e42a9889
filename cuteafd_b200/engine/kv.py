"""Paged KV bookkeeping: a refcounted page pool and per-sequence page lists.

Pages hold 64 tokens.  Refcounts let the prefix cache share the pages of a common prefix between live
sequences and retained snapshots; a page returns to the free list when its last owner releases it.
(Reference: cuteafd-core/src/kv_cache/allocator.rs:12-60, cuteafd-engine/src/prefix/pages.rs.)
"""
from __future__ import annotations

from dataclasses import dataclass, field

PAGE = 64


class OutOfPages(RuntimeError):
    pass


class PagePool:
    def __init__(self, n_pages: int, reserved: int = 1):
        """Page 0 is reserved as the scratch target for padded rows."""
        self.n_pages = n_pages
        self.refs = [0] * n_pages
        self.free = list(range(n_pages - 1, reserved - 1, -1))
        self.reserved = reserved

    @property
    def n_free(self) -> int:
        return len(self.free)

    def alloc(self) -> int:
        if not self.free:
            raise OutOfPages("KV page pool exhausted")
        p = self.free.pop()
        self.refs[p] = 1
        return p

    def retain(self, page: int):
        assert self.refs[page] > 0, "retain of a free page"
        self.refs[page] += 1

    def release(self, page: int):
        assert self.refs[page] > 0, "double release"
        self.refs[page] -= 1
        if self.refs[page] == 0:
            self.free.append(page)

    def can_alloc(self, n: int) -> bool:
        return len(self.free) >= n


@dataclass
class SeqKV:
    """One sequence's view of the cache: its pages (in order) and how many tokens are committed."""
    pages: list = field(default_factory=list)
    length: int = 0

    def pages_needed(self, new_len: int) -> int:
        return max(0, -(-new_len // PAGE) - len(self.pages))

    def ensure(self, pool: PagePool, new_len: int):
        for _ in range(self.pages_needed(new_len)):
            self.pages.append(pool.alloc())

    def slot(self, pos: int) -> int:
        return self.pages[pos // PAGE] * PAGE + pos % PAGE

    def release(self, pool: PagePool):
        for p in self.pages:
            pool.release(p)
        self.pages, self.length = [], 0

    def fork_prefix(self, pool: PagePool, n_tokens: int) -> "SeqKV":
        """New sequence sharing the full pages that cover the first n_tokens (n_tokens % PAGE == 0 shares exactly;
        otherwise the partial last page must be copied by the caller - `copy_on_write_tail`)."""
        n_full = n_tokens // PAGE
        child = SeqKV(pages=list(self.pages[:n_full]), length=n_full * PAGE)
        for p in child.pages:
            pool.retain(p)
        return child
