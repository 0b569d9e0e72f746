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


# ------------------------------------------------------------------ small steps with prompt portions


def bare_mixed(singles, portions, tokens, width, num_groups, scratch_pages, page_size):
    g = graphs_mod.MixedGraph.__new__(graphs_mod.MixedGraph)
    g.set_layout(singles, portions, tokens, width, num_groups)
    g._pad = g.padding(scratch_pages, page_size)
    return g


def test_a_mixed_graphs_padding_names_an_empty_sequence_in_the_scratch_page():
    g = bare_mixed(singles=4, portions=2, tokens=32, width=8, num_groups=1, scratch_pages=[40], page_size=16)
    o, flat = g.offsets, g._pad
    assert (g.n, g.S) == (36, 7) and flat.size == g.size
    assert flat[o["q_start"] : o["q_start"] + 8].tolist() == [0, 1, 2, 3, 4, 4, 4, 4]  # four one-token rows, three empty sequences
    assert flat[o["seq_of_token"] : o["seq_of_token"] + 36].tolist() == [0, 1, 2, 3] + [6] * 32  # the rest name the last, empty one
    assert set(flat[o["kv_len"] : o["kv_len"] + 7].tolist()) == {1}
    base = o["groups"]
    assert set(flat[base : base + 36].tolist()) == {40 * 16} and set(flat[base + 36 : base + g.per_group].tolist()) == {40}
    assert set(flat[o["token_src"] : o["token_src"] + 36].tolist()) == {-1}


def test_fill_of_a_mixed_graph_puts_singles_and_portions_in_their_places():
    from dli_b200.engine.batch import gather_host

    m = CacheManager([GroupSpec(64)], 16, 8, enable_prefix_caching=False, watermark=0.0)
    entries = []
    for rid, have, bring, want in ((0, 20, 1, [0]), (1, 0, 19, []), (2, 47, 1, [0]), (3, 5, 3, [0, 2])):
        toks = list(range(10 * rid, 10 * rid + have + bring))
        m.allocate(rid, toks)
        m.mark_computed(rid, have)
        entries.append(StepEntry(rid, toks[have:], want))
    h = gather_host(entries, m, vocab_size=100)  # order: requests 0, 2 (one token each), then 1, 3
    g = bare_mixed(singles=4, portions=2, tokens=32, width=WIDTH_STEP, num_groups=1, scratch_pages=[64], page_size=16)
    flat, o = g.fill(h), g.offsets
    tok = flat[o["token_ids"] : o["token_ids"] + g.n]
    assert tok[:2].tolist() == [20, 67] and tok[4 : 4 + 22].tolist() == list(range(10, 29)) + [35, 36, 37] and set(tok[26:].tolist()) == {0}
    pos = flat[o["positions"] : o["positions"] + g.n]
    assert pos[:2].tolist() == [20, 47] and pos[4 : 4 + 22].tolist() == list(range(19)) + [5, 6, 7]
    seq = flat[o["seq_of_token"] : o["seq_of_token"] + g.n]
    assert seq[:4].tolist() == [0, 1, 2, 3] and seq[4 : 4 + 22].tolist() == [4] * 19 + [5] * 3 and set(seq[26:].tolist()) == {6}
    assert flat[o["q_start"] : o["q_start"] + 8].tolist() == [0, 1, 2, 3, 4, 23, 26, 26]
    assert flat[o["kv_len"] : o["kv_len"] + 7].tolist() == [21, 48, 1, 1, 19, 8, 1]
    # logits come in the caller's order: request 0's token, request 2's, then places 0 and 2 of request 3's portion
    assert flat[o["logit_rows"] : o["logit_rows"] + 4].tolist() == [0, 1, 23, 25]
    base = o["groups"]
    slots = flat[base : base + g.n]
    assert slots[:2].tolist() == h["slots"][0][:2].tolist() and slots[4 : 4 + 22].tolist() == h["slots"][0][2:].tolist()
    assert set(slots[2:4].tolist()) | set(slots[26:].tolist()) == {64 * 16}
    tables = flat[base + g.n : base + g.per_group].reshape(g.S, WIDTH_STEP)
    assert tables[0, :2].tolist() == m.block_table(0, 0) and tables[4, :2].tolist() == m.block_table(1, 0) and tables[5, :1].tolist() == m.block_table(3, 0)
    assert set(tables[2].tolist()) == set(tables[3].tolist()) == set(tables[6].tolist()) == {64}
    assert np.array_equal(g._pad, bare_mixed(4, 2, 32, WIDTH_STEP, 1, [64], 16)._pad)


def test_mixed_shapes_are_captured_when_they_keep_coming_and_thrashing_shapes_wait_longer(monkeypatch):
    made = []

    class Recorded:
        def __init__(self, model, caches, num_groups, scratch_pages, page_size, singles, portions, tokens, width, launch_keys, pool=None):
            self.shape = (singles, portions, tokens, width)
            made.append(self.shape)

    monkeypatch.setattr(graphs_mod, "MixedGraph", Recorded)
    monkeypatch.setattr(graphs_mod.torch.cuda, "graph_pool_handle", lambda: "pool")
    model = SimpleNamespace(parts=lambda: [], device="cpu")
    pools = SimpleNamespace(layer_caches=[], group_needs=[None], scratch_pages=[7])
    graphs = DecodeGraphs(model, pools, page_size=16)
    assert graphs.mixed_after >= 8  # a capture costs many steps
    graphs.mixed_after = 2
    assert graphs.lookup_mixed(3, 1, 100, 10, 4) is None and made == []  # the first time: launched kernel by kernel
    g = graphs.lookup_mixed(8, 2, 128, 60, 5)  # the same buckets
    assert g.shape == (8, 4, 128, 64) and graphs.lookup_mixed(3, 1, 70, 1, 1) is g and len(made) == 1
    assert graphs.lookup_mixed(0, 3, 1024, 100, 4) is None  # no single tokens, a table 128 pages wide: its own shape
    assert graphs.lookup_mixed(0, 3, 1000, 65, 4).shape == (0, 4, 1024, 128)
    assert graphs.lookup_mixed(3, 1, 100, 10, 13) is None  # more logits wanted than the graph returns rows (8 + 4)
    assert graphs.lookup_mixed(3, 5, 100, 10, 1) is None and graphs.lookup_mixed(3, 1, 1025, 10, 1) is None  # outside the buckets
    graphs.max_mixed = 1
    for _ in range(2):
        other = graphs.lookup_mixed(16, 1, 16, 10, 1)
    assert other.shape == (16, 4, 32, 64) and list(graphs.mixed) == [(16, 4, 32, 64, ())]  # both earlier graphs made room
    first = (8, 4, 128, 64, ())
    assert graphs._needed[first] == 4  # the shape that made room must now come four times
    assert [graphs.lookup_mixed(4, 1, 128, 60, 5) for _ in range(3)] == [None] * 3 and graphs.lookup_mixed(4, 1, 128, 60, 5) is not None


def test_which_steps_are_small_enough_to_be_replayed():
    from dli_b200.engine.runner import ModelRunner

    small = ModelRunner._small_mixed_step
    one = lambda i: StepEntry(i, [5], [0])
    portion = lambda i, n: StepEntry(i, list(range(n)), [n - 1])
    assert not small([one(0), one(1)])  # single tokens only: the decode graphs' business
    assert small([portion(0, 2)]) and small([one(0), portion(1, 1024)]) and small([portion(i, 256) for i in range(4)])
    assert not small([portion(0, 1025)]) and not small([portion(i, 300) for i in range(4)])  # more tokens than the largest bucket
    assert not small([portion(i, 3) for i in range(5)])  # more portions than a graph has places for
    assert small([one(i) for i in range(256)] + [portion(300, 16)]) and not small([one(i) for i in range(257)] + [portion(300, 16)])
