"""The host side of the captured decode steps: buckets, the static buffer's layout, padding rows.  No GPU
(a DecodeGraph is made without its constructor, which captures on the device)."""

import numpy as np

from dli_b200.cache import CacheManager, GroupSpec
from dli_b200.engine import StepEntry
from dli_b200.engine.batch import gather_single_tokens
from types import SimpleNamespace

from dli_b200.engine import graphs as graphs_mod
from dli_b200.engine.graphs import SEQ_BUCKETS, WIDTH_STEP, DecodeGraph, DecodeGraphs, bucket_seqs


def bare_graph(seqs, width, num_groups, scratch_pages, page_size):
    g = DecodeGraph.__new__(DecodeGraph)
    g.seqs, g.width, g.num_groups = seqs, width, num_groups
    per_group = seqs + seqs * width
    g.src_base = 4 * seqs + num_groups * per_group
    g.size = g.src_base + seqs
    g._pad = g.padding(scratch_pages, page_size)
    return g


def test_buckets():
    assert [bucket_seqs(n) for n in (1, 2, 3, 8, 9, 64, 65, 256)] == [1, 2, 4, 8, 16, 64, 96, 256]
    assert bucket_seqs(257) is None and list(SEQ_BUCKETS) == sorted(SEQ_BUCKETS) and WIDTH_STEP % 8 == 0


def test_padding_rows_live_in_the_scratch_page():
    g = bare_graph(seqs=4, width=8, num_groups=2, scratch_pages=[40, 30], page_size=16)
    flat = g._pad
    assert flat.size == g.size and flat[0:4].tolist() == [0] * 4 and flat[4:8].tolist() == [0] * 4  # token 0 at position 0
    assert flat[8:12].tolist() == [1] * 4  # a sequence of one token
    for grp, page in enumerate((40, 30)):
        base = 16 + grp * (4 + 32)
        assert flat[base : base + 4].tolist() == [page * 16] * 4  # written into the scratch page
        assert set(flat[base + 4 : base + 36].tolist()) == {page}  # and read from it
    assert flat[g.src_base :].tolist() == [-1] * 4  # no row takes its token from the device


def test_fill_puts_a_gathered_step_in_front_of_the_padding():
    m = CacheManager([GroupSpec(64), GroupSpec(64)], 16, 8, enable_prefix_caching=False, watermark=0.0)
    entries = []
    for i, have in enumerate((20, 3, 47)):
        toks = list(range(have + 1))
        m.allocate(i, toks)
        m.mark_computed(i, have)
        entries.append(StepEntry(i, [0] if i == 1 else toks[-1:], [0], token_src=5 if i == 1 else -1))
    h = gather_single_tokens(entries, m, vocab_size=100)
    g = bare_graph(seqs=4, width=WIDTH_STEP, num_groups=2, scratch_pages=[64, 64], page_size=16)
    flat = g.fill(h)
    S, seqs, width = 3, 4, WIDTH_STEP
    assert flat[0:S].tolist() == [20, 0, 47] and flat[S] == 0  # the fourth row is padding
    assert flat[seqs : seqs + S].tolist() == [20, 3, 47] and flat[2 * seqs : 2 * seqs + 4].tolist() == [21, 4, 48, 1]
    assert flat[3 * seqs : 3 * seqs + S].tolist() == [m.state_slot(i) for i in range(3)]
    for grp in range(2):
        base = 4 * seqs + grp * (seqs + seqs * width)
        assert flat[base : base + S].tolist() == h["slots"][grp].tolist() and flat[base + S] == 64 * 16
        tables = flat[base + seqs : base + seqs + seqs * width].reshape(seqs, width)
        for i in range(3):
            table = m.block_table(i, grp)
            assert tables[i, : len(table)].tolist() == table and set(tables[i, h["width"] :].tolist()) == {64}
        assert set(tables[3].tolist()) == {64}
    assert flat[g.src_base : g.src_base + 4].tolist() == [-1, 5, -1, -1]
    assert np.array_equal(g._pad, bare_graph(4, WIDTH_STEP, 2, [64, 64], 16)._pad), "fill must not write into the padding it starts from"


def test_graphs_are_keyed_by_what_the_parts_answer_and_the_stalest_one_makes_room(monkeypatch):
    """The graph layer imports no kernel policy: it asks every part of the model what changes its launches, keys
    a shape's graph by the answers, and hands them to the graph (which puts them in its batch).  At the cap the
    least recently used graph goes, so a long run whose shapes drift keeps recording."""
    made = []

    class Recorded:
        def __init__(self, model, caches, num_groups, scratch_pages, page_size, seqs, width, launch_keys):
            self.shape, self.launch_keys = (seqs, width), dict(launch_keys)
            made.append(self)

    monkeypatch.setattr(graphs_mod, "DecodeGraph", Recorded)

    class Splitter:
        def decode_launch_key(self, num_seqs, max_kv_len, page_size):
            return max(1, min(8, max_kv_len // (1024 * num_seqs)))

    class Indifferent:  # has the method's default answer
        def decode_launch_key(self, num_seqs, max_kv_len, page_size):
            return None

    class Unaware:  # a part from before the method existed
        pass

    a, b = Splitter(), Splitter()
    model = SimpleNamespace(parts=lambda: [a, Indifferent(), Unaware(), b], device="cpu")
    pools = SimpleNamespace(layer_caches=[], group_needs=[None], scratch_pages=[7])
    graphs = DecodeGraphs(model, pools, page_size=16)
    g1 = graphs.lookup(3, 10, 150)  # 4 rows, 64 pages = 1,024 keys
    assert g1.shape == (4, 64) and g1.launch_keys == {id(a): 1, id(b): 1} and list(graphs.graphs) == [(4, 64, (1, 1))]
    assert graphs.lookup(4, 60, 900) is g1 and len(made) == 1
    g2 = graphs.lookup(1, 200, 3100)  # 1 row, 256 pages = 4,096 keys: four runs
    assert g2.launch_keys == {id(a): 4, id(b): 4} and (1, 256, (4, 4)) in graphs.graphs
    graphs.max_graphs = 2
    assert graphs.lookup(3, 12, 100) is g1  # used again: g2 is now the stalest
    g3 = graphs.lookup(8, 10, 100)
    assert g3 is not None and list(graphs.graphs) == [(4, 64, (1, 1)), (8, 64, (1, 1))], "the least recently used graph makes room"
    assert graphs.lookup(300, 10, 100) is None  # more rows than the largest bucket: step by step
