"""The cache manager against the reference's own block manager: the operations of
tests/golden/cache_trace.json (made by tests/golden/make_cache_trace.py from
``dli.kv.block_manager.BlockManager``) are run here and every answer and counter is compared:
which admissions are refused, how many tokens the prefix index supplies, which pages a table
holds, which pages are copied for a fork, what is evicted, and what two probes would get.  No GPU."""

import json
from pathlib import Path

import pytest

from dli_b200.cache import CacheManager, GroupSpec, OutOfPages

CASES = json.loads((Path(__file__).resolve().parent / "golden" / "cache_trace.json").read_text())


def observe(m, probes):
    """The same row of counters as ``observe`` of tests/golden/make_cache_trace.py."""
    snap = m.stats()
    g = snap.groups[0]
    row = [g.free_pages, g.cached_idle_pages, g.used_pages, g.evictions, snap.prompt_tokens_queried, snap.prompt_tokens_hit,
           snap.page_copies, g.duplicate_registrations, m.min_available_pages()]
    for p in probes:
        row += [int(m.can_allocate(p)), m.pages_needed_for_prompt(p)]
    return row


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c['policy']}-{c['num_blocks']}x{c['block_size']}-seed{c['seed']}")
def test_same_answers_as_the_reference(case):
    m = CacheManager([GroupSpec(case["num_blocks"])], case["block_size"], max_requests=512, watermark=case["watermark"],
                     eviction_policy=case["policy"])
    live = set()
    for i, rec in enumerate(case["ops"]):
        what = f"operation {i}: {rec['op']}"
        if rec["op"] == "allocate":
            try:
                alloc = m.allocate(rec["id"], rec["tokens"], respect_watermark=rec["respect_watermark"])
                assert not rec.get("fails"), f"{what} was refused by the reference"
                assert alloc.num_cached_tokens == rec["cached"], what
                live.add(rec["id"])
            except OutOfPages:
                assert rec.get("fails"), f"{what} was accepted by the reference"
        elif rec["op"] == "append":
            try:
                copies = m.append_slots(rec["id"], rec["tokens"])
                assert not rec.get("fails"), f"{what} was refused by the reference"
                assert [[c.src, c.dst] for c in copies] == rec["copies"], what
            except OutOfPages:
                assert rec.get("fails"), f"{what} was accepted by the reference"
        elif rec["op"] == "compute":
            m.mark_computed(rec["id"], rec["n"])
        elif rec["op"] == "free":
            m.free(rec["id"])
            live.discard(rec["id"])
        elif rec["op"] == "fork":
            m.fork(rec["parent"], rec["child"])
            live.add(rec["child"])
        elif rec["op"] == "reset":
            assert m.reset_prefix_cache() == rec["evicted"], what
        m.check_invariants()
        assert observe(m, case["probes"]) == rec["after"], what
        if "tables" in rec:
            assert {rid: m.block_table(rid) for rid in sorted(live)} == rec["tables"], what
