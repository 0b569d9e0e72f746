"""The cache manager: block tables per request and group, and per-request state slots.

It holds metadata only (the bytes live in ``cache.pools``).  Layers whose mixers
have equal needs form a *group*; each group has pages of its own (its own page
ids) and each request has one block table per group.  A group with a window
gives a page back as soon as every position in it is older than the window
(the table keeps ``-1`` there).  Beside the pages, each live request holds one
*state slot*, an index into per-layer tensors of fixed-size state.

Calls mirror src/dli/kv/block_manager.py (allocate :238, append_slots :286,
mark_computed :322, free :360, slot_mapping :204, check_invariants :384): a call
that cannot get its pages raises ``OutOfPages`` before it changes anything.
Prefix reuse (hash-chained full pages) works when every group keeps all keys;
with a windowed group, or with mixers that hold state, a prefix's pages alone
do not restore a request, so reuse is off.
"""

from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np

from .page_pool import ROOT, OutOfPages, PagePool, chain_hashes, page_hash

UNKNOWN_TOKEN = -1  # stands for a token id that is still on the device (append_slots, set_token)


class UnknownRequest(KeyError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    """One cache group: how many pages it has and whether it keeps a window only."""

    num_pages: int
    window: int | None = None


@dataclass(frozen=True)
class Allocation:
    num_cached_tokens: int  # leading tokens whose keys and values are already in pages
    state_slot: int


@dataclass
class CacheStats:
    """Counters since construction.  Calling the object (``manager.stats()``, the reference's
    spelling: src/dli/kv/block_manager.py:84-105,222-234) gives a snapshot that also holds the
    pages' states, per cache group."""

    prompt_tokens_queried: int = 0
    prompt_tokens_hit: int = 0
    page_copies: int = 0  # copy-on-write of a forked request's last page
    _pools: list = field(default_factory=list, repr=False)

    @property
    def hit_rate(self) -> float:
        return self.prompt_tokens_hit / self.prompt_tokens_queried if self.prompt_tokens_queried else 0.0

    def __call__(self) -> "CacheSnapshot":
        groups = [GroupPages(p.num_pages, len(p.free), p.num_idle, p.num_pages - len(p.free) - p.num_idle, p.evictions,
                             p.duplicate_registrations) for p in self._pools]
        return CacheSnapshot(self.prompt_tokens_queried, self.prompt_tokens_hit, self.hit_rate, self.page_copies, groups)


@dataclass(frozen=True)
class GroupPages:
    """Pages of one cache group by state: free, idle in the prefix index (evictable in the end), used."""

    num_pages: int
    free_pages: int
    cached_idle_pages: int
    used_pages: int
    evictions: int
    duplicate_registrations: int


@dataclass(frozen=True)
class CacheSnapshot:
    prompt_tokens_queried: int
    prompt_tokens_hit: int
    hit_rate: float
    page_copies: int
    groups: list[GroupPages]


@dataclass(frozen=True)
class PageCopy:
    """Copy page ``src`` to page ``dst`` in every layer of cache group ``group``."""

    group: int
    src: int
    dst: int


@dataclass
class _Request:
    tables: list[list[int]]  # per group: page of block j, or -1 once the window passed it
    num_tokens: int
    num_computed: int
    namespace: bytes
    slot: int
    hashes: list[bytes] = field(default_factory=list)  # chain over the leading full pages known so far
    tail: list[int] = field(default_factory=list)  # tokens after the hashed ones
    registered: int = 0  # leading pages already indexed or taken from the index


class CacheManager:
    def __init__(
        self,
        groups: Sequence[GroupSpec],
        page_size: int,
        max_requests: int,
        *,
        enable_prefix_caching: bool = True,
        has_state: bool = False,
        watermark: float = 0.01,
        eviction_policy: str = "lru",
        debug_checks: bool = False,
    ) -> None:
        # The manager is not locked: it belongs to the one thread that runs the engine's loop.
        # With ``debug_checks`` every call that changes it verifies that
        # (src/dli/kv/block_manager.py:177-183,447-449).
        self._owner = threading.get_ident() if debug_checks else None
        if not 0.0 <= watermark < 1.0:
            raise ValueError("watermark must be in [0, 1)")
        if max_requests < 1:
            raise ValueError("max_requests must be positive")
        self.page_size = page_size
        self.groups = list(groups)
        self.prefix_caching = bool(enable_prefix_caching and groups and not has_state and all(g.window is None for g in groups))
        self.pools = [PagePool(g.num_pages, page_size, self.prefix_caching, eviction_policy) for g in groups]
        self._reserve = [int(watermark * g.num_pages) for g in groups]
        self.max_requests = max_requests
        self._has_window = any(g.window is not None for g in groups)
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._requests: dict[Hashable, _Request] = {}
        self.stats = CacheStats(_pools=self.pools)
        # per group, a copy of every live request's block table as rows of one array (row =
        # state slot), so a step's tables and slots are gathered with array operations
        self._mirror = [np.full((max_requests, 16), -1, dtype=np.int32) for _ in groups]

    # ------------------------------------------------------------ queries

    def has_request(self, rid: Hashable) -> bool:
        return rid in self._requests

    def _confine(self) -> None:
        if self._owner is not None and threading.get_ident() != self._owner:
            raise RuntimeError("the cache manager was called from a thread other than the one that made it")

    def _get(self, rid: Hashable) -> _Request:
        try:
            return self._requests[rid]
        except KeyError:
            raise UnknownRequest(f"unknown request {rid!r}") from None

    def num_tokens(self, rid: Hashable) -> int:
        return self._get(rid).num_tokens

    def num_computed_tokens(self, rid: Hashable) -> int:
        return self._get(rid).num_computed

    def progress(self, rid: Hashable) -> tuple[int, int, int]:
        """(tokens computed, tokens with slots, state slot) of a request, in one look-up."""
        req = self._get(rid)
        return req.num_computed, req.num_tokens, req.slot

    def state_slot(self, rid: Hashable) -> int:
        return self._get(rid).slot

    def block_table(self, rid: Hashable, group: int = 0) -> list[int]:
        return list(self._get(rid).tables[group])

    def slot_mapping(self, rid: Hashable, group: int, start: int, end: int) -> list[int]:
        """Flat slot (page * page_size + offset) of positions [start, end)
        (src/dli/kv/block_manager.py:204-210)."""
        req = self._get(rid)
        if not 0 <= start <= end <= req.num_tokens:
            raise ValueError(f"positions [{start}, {end}) outside reserved [0, {req.num_tokens})")
        ps, table = self.page_size, req.tables[group]
        out = []
        for p in range(start, end):
            page = table[p // ps]
            if page < 0:
                raise ValueError(f"position {p} lies in a page the window has given back")
            out.append(page * ps + p % ps)
        return out

    def table_array(self, group: int) -> np.ndarray:
        """[max_requests, width] int32: row ``state_slot`` holds that request's block table
        (valid up to its number of blocks; -1 where a page was given back)."""
        return self._mirror[group]

    def _mirror_write(self, group: int, slot: int, first: int, pages: Sequence[int]) -> None:
        m = self._mirror[group]
        need = first + len(pages)
        if need > m.shape[1]:
            wider = np.full((m.shape[0], max(need, 2 * m.shape[1])), -1, dtype=np.int32)
            wider[:, : m.shape[1]] = m
            self._mirror[group] = m = wider
        m[slot, first:need] = pages

    def min_available_pages(self) -> int:
        return min((p.available for p in self.pools), default=0)

    def pages_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.page_size)

    def fits_at_all(self, num_tokens: int) -> bool:
        """Whether a request of this many tokens could ever hold its pages, running alone."""
        return all(self.pages_for(num_tokens) <= g.num_pages for g in self.groups)

    # ------------------------------------------------------------ life of a request

    def _hits(self, token_ids: Sequence[int], namespace: bytes) -> tuple[list[list[int]], list[bytes]]:
        """Per group the pages of the longest indexed prefix, never covering the last token:
        a step must run at least one token to give logits (src/dli/kv/block_manager.py:451-465)."""
        if not self.prefix_caching:
            return [[] for _ in self.pools], []
        eligible = (len(token_ids) - 1) // self.page_size * self.page_size
        hashes = chain_hashes(namespace, token_ids[:eligible], self.page_size)
        per_group = [pool.lookup(hashes) for pool in self.pools]
        n = min(len(h) for h in per_group)
        return [h[:n] for h in per_group], hashes

    def _admissible(self, num_tokens: int, hits: list[list[int]], respect_watermark: bool) -> bool:
        if not self._free_slots:
            return False
        need = self.pages_for(num_tokens)
        for pool, h, reserve in zip(self.pools, hits, self._reserve):
            revived = sum(1 for page in h if pool.ref[page] == 0)  # idle hits stop being evictable
            if pool.available - revived - (need - len(h)) < (reserve if respect_watermark else 0):
                return False
        return True

    def pages_needed_for_prompt(self, token_ids: Sequence[int], namespace: bytes = b"") -> int:
        """New pages per group that ``allocate`` would take for this prompt, after prefix hits
        (src/dli/kv/block_manager.py:212-215)."""
        hits, _ = self._hits(token_ids, namespace)
        return self.pages_for(len(token_ids)) - (len(hits[0]) if hits else 0)

    def can_allocate(self, token_ids: Sequence[int], namespace: bytes = b"", respect_watermark: bool = True) -> bool:
        hits, _ = self._hits(token_ids, namespace)
        return self._admissible(len(token_ids), hits, respect_watermark)

    def allocate(self, rid: Hashable, token_ids: Sequence[int], *, namespace: bytes = b"", respect_watermark: bool = True) -> Allocation:
        """Admit a request: pages for all its tokens in every group (indexed prefix pages are
        shared, the rest are taken), and a state slot."""
        self._confine()
        if rid in self._requests:
            raise ValueError(f"request {rid!r} already holds pages")
        if not token_ids:
            raise ValueError("cannot allocate an empty prompt")
        hits, hashes = self._hits(token_ids, namespace)
        if not self._admissible(len(token_ids), hits, respect_watermark):
            raise OutOfPages(f"{self.pages_for(len(token_ids))} pages needed, {self.min_available_pages()} available, "
                             f"{len(self._free_slots)} state slots free")
        tables = []
        for pool, h in zip(self.pools, hits):
            for page in h:  # revive hits before taking pages, so eviction cannot pick them
                pool.share(page)
            tables.append(list(h) + [pool.take() for _ in range(self.pages_for(len(token_ids)) - len(h))])
        n_hit = len(hits[0]) if hits else 0
        cached = n_hit * self.page_size
        self.stats.prompt_tokens_queried += len(token_ids)
        self.stats.prompt_tokens_hit += cached
        req = _Request(tables, len(token_ids), cached, namespace, self._free_slots.pop())
        if self.prefix_caching:
            req.hashes = hashes
            req.tail = list(token_ids[len(hashes) * self.page_size :])
            req.registered = n_hit
        self._requests[rid] = req
        for g, table in enumerate(tables):
            self._mirror_write(g, req.slot, 0, table)
        return Allocation(cached, req.slot)

    def append_slots(self, rid: Hashable, token_ids: Sequence[int]) -> list[PageCopy]:
        """Room for tokens appended to the request (a sampled token); ignores the watermark.
        A token whose id is not known yet (sampled on the device, not read) is UNKNOWN_TOKEN;
        ``set_token`` names it later, and no page that holds one is indexed until then.
        If the request's last page is partly filled and shared with a fork, the request gets a page
        of its own first: the returned copies must be carried out before the step that writes the
        new tokens (src/dli/kv/block_manager.py:286-320)."""
        self._confine()
        req = self._get(rid)
        ps = self.page_size
        first, last = req.num_tokens, req.num_tokens + len(token_ids)
        need = -(-last // ps) - -(-first // ps)  # positions in [first, last) that open a page
        shared = [g for g, (pool, table) in enumerate(zip(self.pools, req.tables))
                  if token_ids and first % ps and table[-1] >= 0 and pool.ref[table[-1]] > 1]
        if any(need + (g in shared) > pool.available for g, pool in enumerate(self.pools)):
            raise OutOfPages(f"append needs {need + bool(shared)} pages")
        copies = []
        for g in shared:
            pool, table = self.pools[g], req.tables[g]
            old, new = table[-1], pool.take()
            pool.release(old)
            table[-1] = new
            self._mirror_write(g, req.slot, len(table) - 1, [new])
            copies.append(PageCopy(g, old, new))
            self.stats.page_copies += 1
        if need:
            for g, (pool, table) in enumerate(zip(self.pools, req.tables)):
                new = [pool.take() for _ in range(need)]
                self._mirror_write(g, req.slot, len(table), new)
                table.extend(new)
        req.num_tokens += len(token_ids)
        if self.prefix_caching:
            req.tail.extend(token_ids)
        return copies

    def fork(self, parent: Hashable, child: Hashable) -> None:
        """A second request that shares every page of ``parent`` (several continuations of one
        prompt).  The first append into the shared, partly filled last page gives the appender a
        page of its own (src/dli/kv/block_manager.py:338-359)."""
        self._confine()
        src = self._get(parent)
        if child in self._requests:
            raise ValueError(f"request {child!r} already holds pages")
        if not self._free_slots:
            raise OutOfPages("no state slot free")
        for pool, table in zip(self.pools, src.tables):
            for page in table:
                if page >= 0:
                    pool.share(page, found_by_hash=False)
        req = _Request([list(t) for t in src.tables], src.num_tokens, src.num_computed, src.namespace, self._free_slots.pop(),
                       list(src.hashes), list(src.tail), src.registered)
        for g, table in enumerate(req.tables):
            self._mirror_write(g, req.slot, 0, table)
        self._requests[child] = req

    def mark_computed(self, rid: Hashable, num_computed: int) -> None:
        """Keys and values of the first ``num_computed`` tokens are written: full pages become
        shareable, and windowed groups give back the pages no later token can read."""
        self._confine()
        req = self._get(rid)
        if not req.num_computed <= num_computed <= req.num_tokens:
            raise ValueError(f"computed must be in [{req.num_computed}, {req.num_tokens}], got {num_computed}")
        req.num_computed = num_computed
        ps = self.page_size
        self._index_full_pages(req)
        if not self._has_window:
            return
        for g, (group, pool, table) in enumerate(zip(self.groups, self.pools, req.tables)):
            if group.window is None:
                continue
            # the next query sits at position >= num_computed and reads keys > position - window
            dead_pages = max(0, (num_computed - group.window + 1) // ps)
            for j in range(min(dead_pages, len(table))):
                if table[j] >= 0:
                    pool.release(table[j])
                    table[j] = -1
                    self._mirror[g][req.slot, j] = -1

    def _index_full_pages(self, req: _Request) -> None:
        """Full pages whose keys and values are written and whose tokens are all known become shareable."""
        ps = self.page_size
        if not self.prefix_caching or req.registered >= req.num_computed // ps:
            return
        full = req.num_computed // ps
        while req.registered < full:
            i = req.registered
            if len(req.hashes) <= i:
                if UNKNOWN_TOKEN in req.tail[:ps]:
                    return  # waits for set_token
                req.hashes.append(page_hash(req.namespace, req.hashes[-1] if req.hashes else ROOT, req.tail[:ps]))
                del req.tail[:ps]
            for pool, table in zip(self.pools, req.tables):
                pool.register(table[i], req.hashes[i], req.hashes[i - 1] if i else None, table[i - 1] if i else None)
            req.registered += 1

    def set_token(self, rid: Hashable, position: int, token_id: int) -> None:
        """Name the token at ``position`` that was appended as UNKNOWN_TOKEN."""
        self._confine()
        req = self._get(rid)
        if not self.prefix_caching:
            return
        i = position - len(req.hashes) * self.page_size
        if not 0 <= i < len(req.tail) or req.tail[i] != UNKNOWN_TOKEN:
            raise ValueError(f"request {rid!r} has no unknown token at position {position}")
        req.tail[i] = int(token_id)
        self._index_full_pages(req)

    def free(self, rid: Hashable) -> None:
        """Give back everything a finished, aborted or preempted request holds."""
        self._confine()
        req = self._requests.pop(rid, None)
        if req is None:
            raise UnknownRequest(f"unknown request {rid!r}")
        for pool, table in zip(self.pools, req.tables):
            for page in reversed(table):  # deepest first: children become evictable before parents
                if page >= 0:
                    pool.release(page)
        self._free_slots.append(req.slot)

    def reset_prefix_cache(self) -> int:
        self._confine()
        return sum(pool.drop_index() for pool in self.pools)

    # ------------------------------------------------------------ verification

    def check_invariants(self) -> None:
        """No page lost, held twice without a count, or freed twice; slots likewise."""
        slots = [r.slot for r in self._requests.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert not set(slots) & set(self._free_slots), "a state slot is both held and free"
        assert len(slots) + len(self._free_slots) == self.max_requests, "a state slot is lost"
        assert len(set(self._free_slots)) == len(self._free_slots), "a state slot is free twice"
        for g, pool in enumerate(self.pools):
            expected: dict[int, int] = {}
            for req in self._requests.values():
                table = req.tables[g]
                assert len(table) == self.pages_for(req.num_tokens), "table size != ceil(tokens / page_size)"
                assert 0 <= req.num_computed <= req.num_tokens
                for j, page in enumerate(table):
                    if page >= 0:
                        expected[page] = expected.get(page, 0) + 1
                    else:
                        w = self.groups[g].window
                        assert w is not None and (j + 1) * self.page_size - 1 <= req.num_computed - w, \
                            "a page still inside the window was given back"
                assert self._mirror[g][req.slot, : len(table)].tolist() == table, "the table array differs from the table"
            pool.check(expected)
