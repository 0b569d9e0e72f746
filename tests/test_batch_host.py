"""The host side of a step's batch: the integer arrays gathered from the cache manager's tables,
against a per-token restatement with the manager's own look-ups.  No GPU."""

import random

import numpy as np
import pytest

from dli_b200.cache import CacheManager, GroupSpec
from dli_b200.engine import StepEntry
from dli_b200.engine.batch import gather_host, gather_single_tokens

VOCAB = 97


def make_requests(rng, manager, count):
    """Requests at different points of their lives: some computed part of their prompt, some
    decoding; returns rid -> tokens that come next (already given slots)."""
    nxt = {}
    for i in range(count):
        rid = f"r{i}"
        have = rng.randrange(0, 23)  # tokens already computed
        more = rng.choice([1, 1, 2, 5, 9])  # tokens of this step
        tokens = [rng.randrange(VOCAB) for _ in range(have + more)]
        manager.allocate(rid, tokens)
        manager.mark_computed(rid, have)
        nxt[rid] = tokens[have:]
    return nxt


@pytest.mark.parametrize("seed", range(6))
def test_gather_host_equals_a_per_token_restatement(seed):
    rng = random.Random(seed)
    ps = rng.choice([1, 4, 16])
    m = CacheManager([GroupSpec(400), GroupSpec(400)], ps, 8, enable_prefix_caching=False, watermark=0.0)
    nxt = make_requests(rng, m, rng.randrange(1, 6))
    entries = []
    for rid, toks in nxt.items():
        want = sorted(rng.sample(range(len(toks)), rng.randrange(0, min(3, len(toks)) + 1)))
        entries.append(StepEntry(rid, toks, want))
    rng.shuffle(entries)
    h = gather_host(entries, m, VOCAB)
    order = [e for e in entries if len(e.token_ids) == 1] + [e for e in entries if len(e.token_ids) != 1]  # single tokens first
    toks, pos, seq, kv, slot_rows, q_start = [], [], [], [], [], [0]
    for s, e in enumerate(order):
        start = m.num_computed_tokens(e.request_id)
        toks += e.token_ids
        pos += list(range(start, start + len(e.token_ids)))
        seq += [s] * len(e.token_ids)
        kv.append(start + len(e.token_ids))
        slot_rows.append(m.state_slot(e.request_id))
        q_start.append(q_start[-1] + len(e.token_ids))
    assert h["n"] == len(toks) and h["S"] == len(order)
    for key, want in (("token_ids", toks), ("positions", pos), ("seq_of_token", seq), ("kv_len", kv), ("state_slot", slot_rows), ("q_start", q_start)):
        assert h[key].tolist() == want, key
    width = -(-max(kv) // ps)
    assert h["width"] == width
    for g in range(2):
        want_slots = [x for e in order for x in m.slot_mapping(e.request_id, g, m.num_computed_tokens(e.request_id), m.num_computed_tokens(e.request_id) + len(e.token_ids))]
        assert h["slots"][g].tolist() == want_slots
        for s, e in enumerate(order):
            table = m.block_table(e.request_id, g)
            assert h["tables"][g][s, : len(table)].tolist()[:width] == table[:width]
    # logits rows: in the order of the entries as given and of their want lists
    first_row = {e.request_id: q_start[s] for s, e in enumerate(order)}
    assert h["logit_rows"].tolist() == [first_row[e.request_id] + w for e in entries for w in e.want]
    assert h["token_src"] is None


@pytest.mark.parametrize("seed", range(4))
def test_single_token_gather_equals_the_general_one(seed):
    rng = random.Random(100 + seed)
    m = CacheManager([GroupSpec(300)], 4, 8, enable_prefix_caching=False, watermark=0.0)
    entries = []
    for i in range(rng.randrange(1, 8)):
        have = rng.randrange(0, 40)
        tokens = [rng.randrange(VOCAB) for _ in range(have + 1)]
        m.allocate(i, tokens)
        m.mark_computed(i, have)
        from_device = rng.random() < 0.4
        entries.append(StepEntry(i, [0] if from_device else tokens[-1:], [0] if rng.random() < 0.8 else [], token_src=i if from_device else -1))
    a, b = gather_host(entries, m, VOCAB), gather_single_tokens(entries, m, VOCAB)
    for key in ("token_ids", "positions", "kv_len", "state_slot", "logit_rows"):
        assert a[key].tolist() == b[key].tolist(), key
    assert a["width"] == b["width"] and a["S"] == b["S"]
    assert a["slots"][0].tolist() == b["slots"][0].tolist() and (a["tables"][0] == b["tables"][0]).all()
    assert (a["token_src"] is None) == (b["token_src"] is None)
    if a["token_src"] is not None:
        assert a["token_src"].tolist() == b["token_src"].tolist()


def test_refusals_name_the_request():
    m = CacheManager([GroupSpec(40)], 4, 4, enable_prefix_caching=False, watermark=0.0)
    m.allocate("a", [1, 2, 3])
    m.allocate("b", [4])
    ok = StepEntry("a", [1, 2, 3], [2])
    for entries, word in (
        ([], "at least one"),
        ([ok, StepEntry("a", [1], [0])], "twice"),
        ([StepEntry("a", [], [])], "no tokens"),
        ([StepEntry("a", [1, 2, VOCAB], [])], "outside the vocabulary"),
        ([StepEntry("a", [1, -1, 2], [])], "outside the vocabulary"),
        ([StepEntry("a", [1, 2, 3], [3])], "want index"),
        ([StepEntry("a", [1, 2, 3, 4], [])], "no slots reserved"),
        ([StepEntry("a", [1, 2], [], token_src=0)], "comes alone"),
    ):
        with pytest.raises(ValueError, match=word):
            gather_host(entries, m, VOCAB)
    for entries, word in (
        ([], "at least one"),
        ([StepEntry("b", [4], [0]), StepEntry("b", [4], [0])], "twice"),
        ([StepEntry("b", [VOCAB], [0])], "outside the vocabulary"),
        ([StepEntry("b", [4], [1])], "want index"),
    ):
        with pytest.raises(ValueError, match=word):
            gather_single_tokens(entries, m, VOCAB)
    m.mark_computed("b", 1)
    with pytest.raises(ValueError, match="no slots reserved"):
        gather_single_tokens([StepEntry("b", [5], [0])], m, VOCAB)


def test_a_position_in_a_page_the_window_gave_back_is_refused():
    m = CacheManager([GroupSpec(40, window=4)], 4, 2, watermark=0.0)
    tokens = list(range(20))
    m.allocate("w", tokens)
    m.mark_computed("w", 16)  # the first pages are behind the window now
    assert m.block_table("w")[0] == -1
    h = gather_host([StepEntry("w", tokens[16:], [3])], m, VOCAB)
    assert h["positions"].tolist() == [16, 17, 18, 19] and (h["tables"][0][0, :2] == -1).all()
