"""Pages of one cache group: free list, reference counts and the prefix index.

A page is in exactly one state: FREE (on the free list), USED (referenced by
``ref`` block-table entries) or IDLE (``ref == 0`` but registered in the prefix
index: its contents stay valid and a later request with the same prefix can
take it over, or it is evicted when memory is needed).  States and rules follow
src/dli/kv/block_manager.py:9-29: only full pages are indexed, only after their
keys were computed; the index is prefix-closed and only idle pages without an
indexed child are evicted, least recently released first
(src/dli/kv/eviction.py:59-90).
"""

from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict, deque
from dataclasses import dataclass
from typing import Sequence

ROOT = b"\x00" * 32


def page_hash(namespace: bytes, parent: bytes, tokens: Sequence[int]) -> bytes:
    """SHA-256 over (length-prefixed namespace, parent page's hash, tokens as int64):
    a page's hash names its whole prefix (src/dli/kv/hashing.py:33-50)."""
    h = hashlib.sha256()
    h.update(struct.pack("<I", len(namespace)))
    h.update(namespace)
    h.update(parent)
    h.update(struct.pack(f"<{len(tokens)}q", *tokens))
    return h.digest()


def chain_hashes(namespace: bytes, tokens: Sequence[int], page_size: int) -> list[bytes]:
    """Hashes of the full pages of ``tokens``, each chained to the one before."""
    out: list[bytes] = []
    parent = ROOT
    for start in range(0, len(tokens) - page_size + 1, page_size):
        parent = page_hash(namespace, parent, tokens[start : start + page_size])
        out.append(parent)
    return out


class OutOfPages(RuntimeError):
    """Not enough free or evictable pages; nothing was changed."""


@dataclass
class _Indexed:
    digest: bytes
    parent: int | None
    children: int = 0


class PagePool:
    def __init__(self, num_pages: int, page_size: int, prefix_index: bool) -> None:
        if num_pages < 1 or page_size < 1:
            raise ValueError("num_pages and page_size must be positive")
        self.num_pages = num_pages
        self.page_size = page_size
        self.prefix_index = prefix_index
        self.ref = [0] * num_pages
        self.free: deque[int] = deque(range(num_pages))
        self.indexed: dict[int, _Indexed] = {}
        self.by_hash: dict[bytes, int] = {}
        self.num_idle = 0
        # idle pages without an indexed child, oldest release first: the eviction order
        self.evictable: OrderedDict[int, None] = OrderedDict()
        self.evictions = 0
        self.duplicate_registrations = 0

    # ------------------------------------------------------------ queries

    @property
    def available(self) -> int:
        """Pages obtainable now: free plus idle (every idle page is evictable in the end)."""
        return len(self.free) + self.num_idle

    def lookup(self, hashes: Sequence[bytes]) -> list[int]:
        """Pages holding the longest indexed prefix of the chain."""
        hits: list[int] = []
        for h in hashes:
            page = self.by_hash.get(h)
            if page is None:
                break
            hits.append(page)
        return hits

    # ------------------------------------------------------------ reference counts

    def take(self) -> int:
        """A page with ref 1: from the free list, else the least recently released evictable one."""
        if self.free:
            page = self.free.popleft()
        elif self.evictable:
            page, _ = self.evictable.popitem(last=False)
            self._evict(page)
        else:
            raise OutOfPages("no free or evictable page")
        self.ref[page] = 1
        return page

    def share(self, page: int) -> None:
        """One more reference to a used or idle page (a prefix hit)."""
        if self.ref[page] == 0:
            if page not in self.indexed:
                raise AssertionError(f"share of free page {page}")
            self.num_idle -= 1
            self.evictable.pop(page, None)
        self.ref[page] += 1

    def release(self, page: int) -> None:
        if self.ref[page] <= 0:
            raise AssertionError(f"page {page} released more often than taken")
        self.ref[page] -= 1
        if self.ref[page]:
            return
        entry = self.indexed.get(page)
        if entry is None:
            self.free.append(page)
            return
        self.num_idle += 1
        if entry.children == 0:
            self.evictable[page] = None

    def _evict(self, page: int) -> None:
        entry = self.indexed.pop(page)
        del self.by_hash[entry.digest]
        self.num_idle -= 1
        self.evictions += 1
        if entry.parent is not None:
            parent = self.indexed[entry.parent]
            parent.children -= 1
            if parent.children == 0 and self.ref[entry.parent] == 0:
                self.evictable[entry.parent] = None  # the parent is now a leaf

    def drop_index(self) -> int:
        """Evict every idle page (its contents are forgotten).  Returns how many."""
        n = 0
        while self.evictable:
            page, _ = self.evictable.popitem(last=False)
            self._evict(page)
            self.free.append(page)
            n += 1
        return n

    # ------------------------------------------------------------ registration

    def register(self, page: int, digest: bytes, parent_digest: bytes | None, parent_page: int | None) -> None:
        """Index a full, computed page under its hash (src/dli/kv/block_manager.py:530-562).

        Not indexed when the same contents are already indexed in another page (this one stays
        private), or when the parent is not indexed as this sequence's own previous page: an idle
        page must never have an in-use descendant, or ``available`` would count pages that cannot
        be evicted.
        """
        if page in self.indexed:
            return
        if digest in self.by_hash:
            self.duplicate_registrations += 1
            return
        parent = None
        if parent_digest is not None:
            parent = self.by_hash.get(parent_digest)
            if parent is None or parent != parent_page:
                return
            pentry = self.indexed[parent]
            if pentry.children == 0 and self.ref[parent] == 0:
                self.evictable.pop(parent, None)
            pentry.children += 1
        self.indexed[page] = _Indexed(digest, parent)
        self.by_hash[digest] = page

    # ------------------------------------------------------------ verification

    def check(self, expected_ref: dict[int, int]) -> None:
        """Every page in exactly one state, counts equal to table references, index closed."""
        for page in range(self.num_pages):
            assert self.ref[page] == expected_ref.get(page, 0), f"page {page}: ref {self.ref[page]} != {expected_ref.get(page, 0)}"
        free = set(self.free)
        assert len(free) == len(self.free), "a page is on the free list twice"
        used = {p for p in range(self.num_pages) if self.ref[p] > 0}
        indexed = set(self.indexed)
        assert not free & used, "a page is both free and used"
        assert not free & indexed, "a page is both free and indexed"
        assert free | used | indexed == set(range(self.num_pages)), "a page is in no state (lost)"
        idle = indexed - used
        assert len(idle) == self.num_idle, "idle counter drifted"
        assert len(self.by_hash) == len(self.indexed), "hash index size differs"
        children: dict[int, int] = {}
        for page, e in self.indexed.items():
            assert self.by_hash.get(e.digest) == page, f"page {page} not found under its hash"
            if e.parent is not None:
                assert e.parent in self.indexed, f"page {page}: parent not indexed"
                children[e.parent] = children.get(e.parent, 0) + 1
        for page, e in self.indexed.items():
            assert e.children == children.get(page, 0), f"page {page}: child count drifted"
            if page in used:
                assert e.parent is None or self.ref[e.parent] > 0, f"used page {page} has an idle parent"
        leaves = {p for p in idle if self.indexed[p].children == 0}
        assert set(self.evictable) == leaves, "evictable set is not the idle leaves"
