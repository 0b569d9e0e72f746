"""The cache manager: no page lost, held twice or freed twice, under random orders (no GPU)."""

import random

import pytest

from dli_b200.cache import CacheManager, GroupSpec, OutOfPages, UnknownRequest, chain_hashes, page_hash


def make(pages=8, page=4, **kw):
    kw.setdefault("watermark", 0.0)
    return CacheManager([GroupSpec(pages)], page, kw.pop("max_requests", 8), **kw)


def test_allocate_tables_slots_and_free():
    m = make()
    a = m.allocate("a", list(range(10)))
    assert a.num_cached_tokens == 0 and len(m.block_table("a")) == 3
    t = m.block_table("a")
    assert m.slot_mapping("a", 0, 3, 10) == [t[0] * 4 + 3, *[t[1] * 4 + i for i in range(4)], t[2] * 4, t[2] * 4 + 1]
    m.append_slots("a", [1, 2])  # fills the third page
    assert len(m.block_table("a")) == 3
    m.append_slots("a", [3])
    assert len(m.block_table("a")) == 4 and m.num_tokens("a") == 13
    m.check_invariants()
    m.free("a")
    assert m.min_available_pages() == 8
    with pytest.raises(UnknownRequest):
        m.free("a")
    m.check_invariants()


def test_out_of_pages_changes_nothing():
    m = make(pages=4)
    m.allocate("a", list(range(12)))
    with pytest.raises(OutOfPages):
        m.allocate("b", list(range(8)))
    assert not m.has_request("b")
    m.append_slots("a", [0, 0, 0, 0])
    with pytest.raises(OutOfPages):
        m.append_slots("a", [0])
    assert m.num_tokens("a") == 16
    m.check_invariants()


def test_watermark_holds_pages_back_for_running_requests():
    m = CacheManager([GroupSpec(100)], 4, 8, watermark=0.1)
    assert not m.can_allocate(list(range(4 * 91)))
    assert m.can_allocate(list(range(4 * 90)))
    m.allocate("a", list(range(4 * 90)))
    m.append_slots("a", list(range(4 * 10)))  # growth ignores the watermark
    m.check_invariants()


def test_state_slots_are_unique_and_reused():
    m = make(pages=32, max_requests=3)
    slots = [m.allocate(i, [1, 2]).state_slot for i in range(3)]
    assert sorted(slots) == [0, 1, 2]
    assert not m.can_allocate([1])
    with pytest.raises(OutOfPages):
        m.allocate(9, [1])
    m.free(1)
    assert m.allocate(9, [1]).state_slot == slots[1]
    m.check_invariants()


def test_prefix_pages_are_shared_only_after_they_were_computed():
    m = make(pages=16)
    prompt = list(range(100, 110))  # 2 full pages + 2 tokens
    m.allocate("a", prompt)
    assert m.allocate("b", prompt).num_cached_tokens == 0  # nothing computed yet
    m.mark_computed("a", 10)
    m.mark_computed("b", 10)  # same contents in other pages: stays private
    assert m.pools[0].duplicate_registrations == 2
    c = m.allocate("c", prompt + [7, 8, 9])
    assert c.num_cached_tokens == 8 and m.block_table("c")[:2] == m.block_table("a")[:2]
    assert m.num_computed_tokens("c") == 8
    m.check_invariants()
    for r in "abc":
        m.free(r)
    m.check_invariants()
    assert m.pools[0].num_idle == 2  # the two indexed pages stay, revivable
    d = m.allocate("d", prompt[:8])  # the page of the last token is always recomputed
    assert d.num_cached_tokens == 4
    m.check_invariants()


def test_namespace_separates_prefixes():
    assert chain_hashes(b"x", [1, 2, 3, 4], 4) != chain_hashes(b"y", [1, 2, 3, 4], 4)
    assert page_hash(b"ab", b"\0" * 32, [1]) != page_hash(b"a", b"\0" * 32, [1])
    m = make(pages=16)
    m.allocate("a", list(range(9)), namespace=b"m1")
    m.mark_computed("a", 9)
    assert m.allocate("b", list(range(9)), namespace=b"m2").num_cached_tokens == 0
    assert m.allocate("c", list(range(9)), namespace=b"m1").num_cached_tokens == 8


def test_idle_pages_are_evicted_leaf_first_oldest_first():
    m = make(pages=4)
    m.allocate("a", list(range(9)))  # 3 pages, 2 full
    m.mark_computed("a", 9)
    m.free("a")
    assert m.pools[0].num_idle == 2 and m.min_available_pages() == 4
    m.allocate("b", [50] * 13)  # needs all 4: evicts the leaf, then its parent
    assert m.pools[0].evictions == 2
    m.check_invariants()
    m.free("b")
    assert m.allocate("c", list(range(9))).num_cached_tokens == 0


def test_prefix_caching_off():
    m = make(enable_prefix_caching=False)
    m.allocate("a", list(range(9)))
    m.mark_computed("a", 9)
    m.free("a")
    assert m.pools[0].num_idle == 0 and m.allocate("b", list(range(9))).num_cached_tokens == 0


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([GroupSpec(8), GroupSpec(8, window=6)], 4, 4, watermark=0.0)
    assert not m.prefix_caching  # a prefix's pages alone would not restore a windowed group
    m.allocate("a", list(range(14)))
    assert len(m.block_table("a", 0)) == 4 and len(m.block_table("a", 1)) == 4
    m.mark_computed("a", 9)  # next query at >= 9 reads keys > 3: page 0 (keys 0..3) is dead
    assert m.block_table("a", 1)[0] == -1 and m.block_table("a", 1)[1] >= 0
    assert m.pools[1].available == 5 and m.pools[0].available == 4
    m.check_invariants()
    with pytest.raises(ValueError, match="given back"):
        m.slot_mapping("a", 1, 0, 4)
    m.mark_computed("a", 14)  # keys > 8 stay: pages 0 and 1 dead
    assert m.block_table("a", 1)[:2] == [-1, -1]
    m.append_slots("a", [1, 2, 3])
    m.check_invariants()
    m.free("a")
    assert m.pools[1].available == 8 and m.pools[0].available == 8
    m.check_invariants()


def test_mark_computed_is_monotone():
    m = make()
    m.allocate("a", list(range(6)))
    m.mark_computed("a", 4)
    with pytest.raises(ValueError):
        m.mark_computed("a", 3)
    with pytest.raises(ValueError):
        m.mark_computed("a", 7)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("prefix_caching, window", [(True, None), (False, None), (False, 7)])
def test_random_orders_keep_every_invariant(seed, prefix_caching, window):
    """Requests arrive, grow, are computed in portions, finish and are preempted in random
    order.  A shadow store maps every slot to the token prefix written there, so a page held
    twice, freed while in use, or shared with other contents shows as a wrong read."""
    rng = random.Random(seed)
    page = rng.choice([1, 3, 4])
    groups = [GroupSpec(24)] + ([GroupSpec(20, window=window)] if window else [])
    m = CacheManager(groups, page, 5, enable_prefix_caching=prefix_caching, watermark=0.0, eviction_policy=rng.choice(["lru", "cost"]))
    shadow = [dict() for _ in groups]  # per group: slot -> prefix tuple
    tokens: dict[int, list[int]] = {}
    stems = [[rng.randrange(5) for _ in range(12)] for _ in range(3)]
    next_id = 0
    for _ in range(600):
        op = rng.random()
        live = list(tokens)
        if op < 0.25 or not live:
            toks = (rng.choice(stems)[: rng.randrange(1, 13)] if rng.random() < 0.7 else []) + [rng.randrange(5) for _ in range(rng.randrange(1, 9))]
            ok = m.can_allocate(toks)
            try:
                alloc = m.allocate(next_id, toks)
                assert ok
                tokens[next_id] = toks
                # cached tokens must already hold this very prefix
                for g in range(len(groups)):
                    for pos, slot in enumerate(m.slot_mapping(next_id, g, 0, alloc.num_cached_tokens)):
                        assert shadow[g][slot] == tuple(toks[: pos + 1])
                next_id += 1
            except OutOfPages:
                assert not ok
        elif op < 0.45:
            rid = rng.choice(live)
            new = [rng.randrange(5) for _ in range(rng.randrange(1, 4))]
            try:
                m.append_slots(rid, new)
                tokens[rid] += new
            except OutOfPages:
                pass
        elif op < 0.8:
            rid = rng.choice(live)
            done, total = m.num_computed_tokens(rid), m.num_tokens(rid)
            if done < total:
                upto = rng.randrange(done + 1, total + 1)
                for g, grp in enumerate(groups):
                    # reads: every key the window still needs holds this request's prefix
                    lo = 0 if grp.window is None else max(0, done - grp.window + 1)
                    for pos, slot in zip(range(lo, done), m.slot_mapping(rid, g, lo, done)):
                        assert shadow[g][slot] == tuple(tokens[rid][: pos + 1]), "a live slot was overwritten"
                    for pos, slot in zip(range(done, upto), m.slot_mapping(rid, g, done, upto)):
                        shadow[g][slot] = tuple(tokens[rid][: pos + 1])
                m.mark_computed(rid, upto)
        else:
            rid = rng.choice(live)
            m.free(rid)
            del tokens[rid]
        m.check_invariants()
    for rid in list(tokens):
        m.free(rid)
    m.check_invariants()
    for pool in m.pools:
        assert pool.available == pool.num_pages


def test_unknown_token_is_not_indexed_until_named():
    """A token appended before its id is known keeps its page out of the prefix index; once named,
    the page is found by a request with the same tokens."""
    from dli_b200.cache import UNKNOWN_TOKEN

    m = CacheManager([GroupSpec(16)], 4, 4, enable_prefix_caching=True, watermark=0.0)
    m.allocate("a", [1, 2, 3])
    m.mark_computed("a", 3)
    m.append_slots("a", [UNKNOWN_TOKEN])
    m.mark_computed("a", 4)  # the page is full and written, but one id is unknown
    m.check_invariants()
    m.allocate("b", [1, 2, 3, 9, 5])
    assert m.num_computed_tokens("b") == 0
    m.free("b")
    with pytest.raises(ValueError):
        m.set_token("a", 2, 7)  # position 2 is known
    m.set_token("a", 3, 9)
    m.check_invariants()
    m.allocate("c", [1, 2, 3, 9, 5])
    assert m.num_computed_tokens("c") == 4
    m.free("a"), m.free("c")
    m.check_invariants()


def test_cost_policy_keeps_the_prefix_that_is_wanted_often():
    """A shared stem that many requests hit survives a burst of one-off prompts under the "cost"
    policy (its pages have many hits and lie deep in their chain); least-recently-released evicts it."""
    stem = list(range(100, 112))  # three full pages of 4

    def run(policy):
        m = CacheManager([GroupSpec(8)], 4, 4, enable_prefix_caching=True, watermark=0.0, eviction_policy=policy)
        for i in range(4):  # the stem is computed once and found three times
            toks = stem + [i]
            m.allocate(f"s{i}", toks)
            m.mark_computed(f"s{i}", len(toks))
            m.free(f"s{i}")
        for i in range(5):  # one-off prompts of one full page each: 5 more pages than the 5 that are free
            toks = [200 + i] * 4 + [7]
            m.allocate(f"u{i}", toks)
            m.mark_computed(f"u{i}", len(toks))
            m.free(f"u{i}")
            m.check_invariants()
        return m.allocate("again", stem + [9]).num_cached_tokens

    assert run("cost") == 12
    assert run("lru") < 12
    with pytest.raises(ValueError):
        CacheManager([GroupSpec(8)], 4, 4, eviction_policy="random")


def test_fork_shares_pages_and_the_first_append_copies_the_last_one():
    m = make(pages=8)  # page size 4
    m.allocate("a", list(range(6)))  # one full page, one with two tokens
    m.mark_computed("a", 6)
    m.fork("a", "b")
    assert m.block_table("a") == m.block_table("b") and m.state_slot("a") != m.state_slot("b")
    m.check_invariants()
    with pytest.raises(ValueError):
        m.fork("a", "b")
    copies = m.append_slots("b", [40])
    assert len(copies) == 1 and copies[0].src == m.block_table("a")[1] and copies[0].dst == m.block_table("b")[1]
    assert m.block_table("a")[0] == m.block_table("b")[0] and m.block_table("a")[1] != m.block_table("b")[1]
    assert m.append_slots("a", [41]) == []  # the last page is a's own again
    assert m.append_slots("b", [42, 43, 44]) == []  # b fills its page and opens the next
    m.check_invariants()
    m.free("a")
    m.check_invariants()
    m.free("b")
    m.check_invariants()
    assert m.min_available_pages() == 8


def test_fork_without_room_for_the_copy_changes_nothing():
    m = make(pages=2, watermark=0.0)
    m.allocate("a", list(range(6)))
    m.mark_computed("a", 6)
    m.fork("a", "b")
    before = (m.block_table("a"), m.block_table("b"), m.num_tokens("b"))
    with pytest.raises(OutOfPages):
        m.append_slots("b", [9])
    assert (m.block_table("a"), m.block_table("b"), m.num_tokens("b")) == before
    m.check_invariants()


def test_debug_checks_refuse_calls_from_another_thread():
    import threading

    m = CacheManager([GroupSpec(8)], 4, 4, debug_checks=True)
    m.allocate("a", [1, 2, 3])
    caught = []

    def elsewhere():
        for call in (lambda: m.append_slots("a", [4]), lambda: m.free("a"), lambda: m.allocate("b", [1])):
            try:
                call()
            except RuntimeError as e:
                caught.append(str(e))

    t = threading.Thread(target=elsewhere)
    t.start()
    t.join()
    assert len(caught) == 3 and all("thread" in c for c in caught)
    assert m.num_tokens("a") == 3 and not m.has_request("b")  # nothing happened
    m.free("a")  # the owner may
    m.check_invariants()


# ---- mutants: every kind of damage is noticed by check_invariants


def _busy_manager():
    """Two live requests sharing two indexed pages, one finished request whose pages idle in the index."""
    m = CacheManager([GroupSpec(16)], 4, 4, watermark=0.0)
    stem = list(range(8))
    for rid, tail in (("gone", [50, 51, 52, 53, 54]), ("a", [20, 21, 22]), ("b", [30])):
        m.allocate(rid, stem + tail)
        m.mark_computed(rid, len(stem + tail))
    m.free("gone")
    m.check_invariants()
    assert m.pools[0].num_idle >= 1 and m.pools[0].ref[m.block_table("a")[0]] == 2
    return m


def _lose_a_free_page(m):
    m.pools[0].free.pop()


def _free_a_page_twice(m):
    m.pools[0].free.append(m.pools[0].free[0])


def _free_a_page_that_is_held(m):
    m.pools[0].free.append(m.block_table("a")[-1])


def _hold_a_page_twice_without_counting(m):
    m._requests["b"].tables[0][-1] = m.block_table("a")[-1]
    m._mirror[0][m.state_slot("b"), len(m.block_table("b")) - 1] = m.block_table("a")[-1]


def _drop_a_reference(m):
    m.pools[0].ref[m.block_table("a")[0]] -= 1


def _table_of_the_wrong_length(m):
    m._requests["a"].tables[0].append(m.pools[0].take())


def _table_array_out_of_step(m):
    m._mirror[0][m.state_slot("a"), 0] += 1


def _lose_a_state_slot(m):
    m._free_slots.pop()


def _give_a_held_slot_away(m):
    m._free_slots.append(m.state_slot("a"))


def _forget_a_hash(m):
    pool = m.pools[0]
    del pool.by_hash[pool.indexed[m.block_table("a")[1]].digest]


def _miscount_children(m):
    m.pools[0].indexed[m.block_table("a")[0]].children += 1


def _miscount_idle(m):
    m.pools[0].num_idle += 1


def _hide_an_idle_leaf_from_eviction(m):
    pool = m.pools[0]
    pool.evictable.discard(next(iter(pool.evictable.pages())))


def _computed_beyond_tokens(m):
    m._requests["a"].num_computed = m._requests["a"].num_tokens + 1


MUTANTS = [_lose_a_free_page, _free_a_page_twice, _free_a_page_that_is_held, _hold_a_page_twice_without_counting, _drop_a_reference,
           _table_of_the_wrong_length, _table_array_out_of_step, _lose_a_state_slot, _give_a_held_slot_away, _forget_a_hash,
           _miscount_children, _miscount_idle, _hide_an_idle_leaf_from_eviction, _computed_beyond_tokens]


@pytest.mark.parametrize("damage", MUTANTS, ids=lambda f: f.__name__.strip("_"))
def test_check_invariants_notices(damage):
    m = _busy_manager()
    damage(m)
    with pytest.raises(AssertionError):
        m.check_invariants()


def test_double_free_and_release_of_a_free_page_raise_at_once():
    m = _busy_manager()
    m.free("a")
    with pytest.raises(UnknownRequest):
        m.free("a")
    with pytest.raises(AssertionError):
        m.pools[0].release(m.pools[0].free[0])
    m.check_invariants()


def test_stats_snapshot_counts_pages_by_state_and_copies():
    m = _busy_manager()  # two live requests on a shared stem, one finished request idling in the index
    snap = m.stats()
    g = snap.groups[0]
    assert g.num_pages == 16 and g.free_pages + g.cached_idle_pages + g.used_pages == 16
    assert g.cached_idle_pages == m.pools[0].num_idle >= 1 and g.used_pages == sum(1 for r in m.pools[0].ref if r > 0)
    assert snap.prompt_tokens_hit == m.stats.prompt_tokens_hit == 16 and 0 < snap.hit_rate < 1 and snap.page_copies == 0
    stem = list(range(8))
    assert m.pages_needed_for_prompt(stem + [70, 71]) == 1  # two pages of the stem are in the index
    assert m.pages_needed_for_prompt([9] * 10) == 3
    m.fork("a", "a2")
    m.append_slots("a2", [5])  # the shared last page is partly filled: it is copied first
    assert m.stats().page_copies == 1
    m.check_invariants()


def test_page_hashes_equal_the_reference():
    """Chains of page hashes recorded from the reference's dli.kv.hashing.chain_hashes
    (tests/golden/make_config_hash_golden.py): the same bytes here, so a prefix index could be shared."""
    import json
    from pathlib import Path

    golden = json.loads((Path(__file__).parent / "golden" / "config_and_hash.json").read_text())
    for case in golden["hashes"]:
        got = chain_hashes(bytes.fromhex(case["namespace"]), case["tokens"], case["page_size"])
        assert [h.hex() for h in got] == case["chain"]
        assert len(got) == len(case["tokens"]) // case["page_size"]
