"""Pages of one cache group: free list, reference counts and the prefix index.

A page is in exactly one state: FREE (on the free list), USED (referenced by
``ref`` block-table entries) or IDLE (``ref == 0`` but registered in the prefix
index: its contents stay valid and a later request with the same prefix can
take it over, or it is evicted when memory is needed).  States and rules follow
src/dli/kv/block_manager.py:9-29: only full pages are indexed, only after their
keys were computed; the index is prefix-closed and only idle pages without an
indexed child are evicted: least recently released first, or — policy ``"cost"`` —
lowest value first, a page's value growing with the hits it had and with its depth in
its chain (src/dli/kv/eviction.py:59-164).
"""

from __future__ import annotations

import hashlib
import heapq
import itertools
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
    depth: int = 0  # pages before this one in its chain
    hits: int = 1  # times its contents were wanted: once when computed, once per later request that found it


class _OldestFirst:
    """Candidates in the order in which they became evictable."""

    def __init__(self) -> None:
        self._order: OrderedDict[int, None] = OrderedDict()

    def add(self, page: int, entry: _Indexed) -> None:
        self._order[page] = None

    def discard(self, page: int) -> None:
        self._order.pop(page, None)

    def pop(self, indexed: dict[int, _Indexed]) -> int:
        return self._order.popitem(last=False)[0]

    def pages(self) -> set[int]:
        return set(self._order)

    def __len__(self) -> int:
        return len(self._order)


class _LowestValueFirst:
    """Greedy-dual with frequency (the scheme of src/dli/kv/eviction.py:93-164): a candidate's value
    is ``floor + hits * (1 + depth_weight * depth)``; the lowest goes first and its value becomes the
    floor, so pages that stop being hit age against newer ones.  All pages have the same size.  A deep
    page of a chain that was wanted often (a shared system prompt) outlives one-off tails.
    A heap with lazy deletion: an entry counts only while its stamp is the page's current one."""

    def __init__(self, depth_weight: float = 0.05) -> None:
        self.depth_weight = depth_weight
        self.floor = 0.0
        self._heap: list[tuple[float, int, int]] = []  # (value, stamp, page)
        self._stamp: dict[int, int] = {}
        self._stamps = itertools.count()

    def add(self, page: int, entry: _Indexed) -> None:
        stamp = self._stamp[page] = next(self._stamps)
        heapq.heappush(self._heap, (self.floor + entry.hits * (1.0 + self.depth_weight * entry.depth), stamp, page))
        if len(self._heap) > 4 * len(self._stamp) + 64:  # mostly stale entries: rebuild
            self._heap = [e for e in self._heap if self._stamp.get(e[2]) == e[1]]
            heapq.heapify(self._heap)

    def discard(self, page: int) -> None:
        self._stamp.pop(page, None)

    def pop(self, indexed: dict[int, _Indexed]) -> int:
        while self._heap:
            value, stamp, page = heapq.heappop(self._heap)
            if self._stamp.get(page) == stamp:
                del self._stamp[page]
                self.floor = value
                return page
        raise KeyError("no candidate")

    def pages(self) -> set[int]:
        return set(self._stamp)

    def __len__(self) -> int:
        return len(self._stamp)


EVICTION_POLICIES = {"lru": _OldestFirst, "cost": _LowestValueFirst}


class PagePool:
    def __init__(self, num_pages: int, page_size: int, prefix_index: bool, eviction_policy: str = "lru") -> None:
        if num_pages < 1 or page_size < 1:
            raise ValueError("num_pages and page_size must be positive")
        if eviction_policy not in EVICTION_POLICIES:
            raise ValueError(f"eviction_policy must be one of {sorted(EVICTION_POLICIES)}, got {eviction_policy!r}")
        self.num_pages = num_pages
        self.page_size = page_size
        self.prefix_index = prefix_index
        self.ref = [0] * num_pages
        self.free: deque[int] = deque(range(num_pages))
        self.indexed: dict[int, _Indexed] = {}
        self.by_hash: dict[bytes, int] = {}
        self.num_idle = 0
        # idle pages without an indexed child, in the policy's eviction order
        self.evictable = EVICTION_POLICIES[eviction_policy]()
        self.eviction_policy = eviction_policy
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
        elif len(self.evictable):
            page = self.evictable.pop(self.indexed)
            self._evict(page)
        else:
            raise OutOfPages("no free or evictable page")
        self.ref[page] = 1
        return page

    def share(self, page: int, found_by_hash: bool = True) -> None:
        """One more reference to a used or idle page: a prefix hit (which counts towards the page's
        value for the cost-aware policy, as in src/dli/kv/block_manager.py:265-268), or a fork of the
        request that holds it (which does not)."""
        if self.ref[page] == 0:
            if page not in self.indexed:
                raise AssertionError(f"share of free page {page}")
            self.num_idle -= 1
            self.evictable.discard(page)
        entry = self.indexed.get(page)
        if entry is not None and found_by_hash:
            entry.hits += 1
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
            self.evictable.add(page, entry)

    def _evict(self, page: int) -> None:
        entry = self.indexed.pop(page)
        del self.by_hash[entry.digest]
        self.num_idle -= 1
        self.evictions += 1
        if entry.parent is not None:
            parent = self.indexed[entry.parent]
            parent.children -= 1
            if parent.children == 0 and self.ref[entry.parent] == 0:
                self.evictable.add(entry.parent, parent)  # the parent is now a leaf

    def drop_index(self) -> int:
        """Evict every idle page (its contents are forgotten).  Returns how many."""
        n = 0
        while len(self.evictable):
            page = self.evictable.pop(self.indexed)
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
                self.evictable.discard(parent)
            pentry.children += 1
        self.indexed[page] = _Indexed(digest, parent, depth=0 if parent is None else self.indexed[parent].depth + 1)
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
        assert self.evictable.pages() == leaves and len(self.evictable) == len(leaves), "evictable set is not the idle leaves"
