"""Replay at the layer sizes of the benchmark models (few layers, random weights): the kernels
that tiny models never reach — 64-wide heads on the tcgen05 and TMA paths, 128-wide heads,
thousands of features per product, a six-digit vocabulary — against the plain implementation."""

import contextlib
import copy

import numpy as np
import pytest
import torch

import dli_b200
from dli_b200.engine import ModelRunner, StepEntry
from dli_b200.engine.batch import GroupView
from dli_b200.kernels import attention as attn_kernels
from dli_b200.kernels import ops
from dli_b200.weights import write_safetensors
from tests.plain import llama_plain as plain
from tests.util import plain_weights_for, random_tokens

pytestmark = pytest.mark.gpu

LLAMA_1B_2L = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "rms_norm_eps": 1e-5,
}
LLAMA_3B_1L = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 3072,
    "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "vocab_size": 32000,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "rms_norm_eps": 1e-5,
}
SMOLLM2_1L = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152,
    "rope_theta": 130000.0, "tie_word_embeddings": True, "rms_norm_eps": 1e-5,
}


_FOLDERS: dict[str, tuple] = {}


def model_folder(name: str, tmp_path_factory):
    """(config, folder, weights) of a benchmark shape, written once per test run."""
    if name not in _FOLDERS:
        cfg = {"llama_1b": LLAMA_1B_2L, "llama_3b": LLAMA_3B_1L, "smollm2": SMOLLM2_1L}[name]
        path = tmp_path_factory.mktemp(name)
        dli_b200.write_model_dir(path, cfg, seed=7)
        # sharpen attention as the tiny-model tests do
        w = {k: torch.from_numpy(v.copy()) for k, v in plain.read_safetensors(path / "model.safetensors").items()}
        for k in w:
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                w[k] = w[k] * 3.0
        write_safetensors(path / "model.safetensors", w)
        _FOLDERS[name] = (cfg, path, {k: v.numpy() for k, v in w.items()})
    return _FOLDERS[name]


@pytest.fixture(scope="module", params=["llama_1b", "llama_3b", "smollm2"])
def case(request, tmp_path_factory):
    cfg, path, weights = model_folder(request.param, tmp_path_factory)
    tokens = random_tokens(cfg["vocab_size"], 300, seed=3)
    return cfg, path, weights, tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_decode_and_batch_at_real_sizes(case, dtype):
    cfg, path, weights, tokens = case
    want = plain.forward(cfg, plain_weights_for(weights, dtype), tokens)
    scale = float(np.abs(want).max())
    tol = (2e-4 if dtype == "float32" else 5e-2) * max(1.0, scale)
    model = dli_b200.load_model(path, dtype)
    r = ModelRunner(model, num_pages=48, page_size=16, max_requests=4, enable_prefix_caching=False, watermark=0.0)

    def run(rid, cuts, want_rows):
        """Feed ``tokens`` in the given portions; logits of every position."""
        pos, parts = 0, []
        for n in cuts:
            piece = tokens[pos : pos + n]
            if r.manager.has_request(rid):
                r.manager.append_slots(rid, piece)
            else:
                r.manager.allocate(rid, piece)
            parts.append(r.step([StepEntry(rid, piece, range(n))]))
            pos += n
        r.manager.free(rid)
        return torch.cat(parts).cpu().numpy()

    whole = run("w", [300], None)
    err = np.abs(whole - want).max(axis=1)
    assert err.max() <= tol, f"whole: first wrong position {int(np.argmax(err > tol))} (error {err.max():.3g}, tolerance {tol:.3g})"
    cut = run("c", [129, 2, 64, 5, 70] + [1] * 30, None)
    err = np.abs(cut - want).max(axis=1)
    assert err.max() <= tol, f"portions + decode: first wrong position {int(np.argmax(err > tol))} (error {err.max():.3g})"

    # two requests side by side: a decoded token of one beside a portion of the other
    r.manager.allocate("a", tokens[:200])
    r.step([StepEntry("a", tokens[:200], [])])
    r.manager.allocate("b", tokens[:150])
    r.manager.append_slots("a", tokens[200:201])
    out = r.step([StepEntry("b", tokens[:150], [149]), StepEntry("a", tokens[200:201], [0])]).cpu().numpy()
    assert np.abs(out[0] - want[149]).max() <= tol and np.abs(out[1] - want[200]).max() <= tol
    # both decode together (the replayed graph)
    r.manager.append_slots("a", tokens[201:202])
    r.manager.append_slots("b", tokens[150:151])
    out = r.step([StepEntry("a", tokens[201:202], [0]), StepEntry("b", tokens[150:151], [0])]).cpu().numpy()
    assert np.abs(out[0] - want[201]).max() <= tol and np.abs(out[1] - want[150]).max() <= tol
    r.manager.check_invariants()


# ---- what the benchmark runs: contexts of 2,048 and more, 1 / 8 / 64 sequences decoding, 8,000 tokens at head size 128
#
# Over thousands of keys the plain implementation rounds where a bfloat16 model rounds (``bf16_activations``: the
# outputs of products, norms, rope and attention, and the attention's probabilities).  With float32 activations and
# only the weights rounded it lies as far from a bfloat16 run (0.28 at 2,048 tokens, logits up to 5) as the
# tolerance allows in all, which would leave a fault nothing to show itself in; rounded alike, the engine is
# within 0.10.


def worst(got, want):
    diff = np.abs(np.asarray(got, dtype=np.float32) - want)
    return float(diff.max()) if np.isfinite(diff).all() else float("inf")


def runner_with_used_pages(model, **kw):
    """A runner whose pages look used: every key and value holds large finite junk, as a page that another
    request gave back would.  Rows of a half-filled page beyond a sequence's end are never to be read; if a
    kernel reads them (or a table names the wrong page), the junk shows."""
    r = ModelRunner(model, enable_prefix_caching=kw.pop("enable_prefix_caching", False), watermark=0.0, **kw)
    for pool in (*r.pools.k, *r.pools.v):
        pool.fill_(1e4)
    return r


@contextlib.contextmanager
def pages_swapped_in_one_layer(layer_cache, row: int, a: int, b: int):
    """While this is open, the attention of ONE layer reads sequence ``row`` of the step through a block table in
    which the valid page ids at places a and b have changed places (the cache was written through the right
    table).  Nothing is out of range; the layer's keys are merely met in the wrong order, so causal masking
    and the half-filled last page go wrong.  A comparison that still passes has no teeth."""
    real = attn_kernels.paged_attention

    def mutated(out, qkv, cache, batch, *rest, **named):
        if cache.k is not None and cache.k.data_ptr() == layer_cache.k.data_ptr():
            view = batch.group(cache.group)
            tables = view.block_tables.clone()
            tables[row, a], tables[row, b] = view.block_tables[row, b], view.block_tables[row, a]
            batch = copy.copy(batch)
            batch.groups = list(batch.groups)
            batch.groups[cache.group] = GroupView(tables, view.slots)
        return real(out, qkv, cache, batch, *rest, **named)

    attn_kernels.paged_attention = mutated
    try:
        yield
    finally:
        attn_kernels.paged_attention = real


@contextlib.contextmanager
def pages_swapped_in_table(manager, rid, a: int, b: int):
    """The same for steps that run from a captured graph (whose launches cannot be wrapped): two valid page ids of
    one request change places in the cache manager's table array, in every layer, for the steps inside."""
    table = manager.table_array(0)
    row = manager.state_slot(rid)
    table[row, a], table[row, b] = table[row, b], table[row, a]
    try:
        yield
    finally:
        table[row, a], table[row, b] = table[row, b], table[row, a]


@pytest.fixture(scope="module")
def long_1b(tmp_path_factory):
    cfg, path, weights = model_folder("llama_1b", tmp_path_factory)
    tokens = random_tokens(cfg["vocab_size"], 2048 + 24, seed=11)
    rows = sorted(set(range(0, 2048, 9)) | set(range(1960, 2048 + 24)))
    want = dict(zip(rows, plain.forward(cfg, plain_weights_for(weights, "bfloat16"), tokens, rows=rows, bf16_activations=True)))
    tol = 5e-2 * max(1.0, max(float(np.abs(v).max()) for v in want.values()))
    return cfg, path, tokens, want, tol


def test_a_prompt_of_2048_tokens_whole_then_one_sequence_decoding(long_1b):
    """One step of 2,048 tokens (the prefill the benchmark times: two query tiles per CTA, a block table 128 pages
    wide), then the same sequence decoded on through the captured graph of one sequence, whose attention splits
    the keys sixteen ways inside one thread-block cluster."""
    cfg, path, tokens, want, tol = long_1b
    model = dli_b200.load_model(path, "bfloat16")
    r = runner_with_used_pages(model, num_pages=(2048 + 64) // 16 + 2, page_size=16, max_requests=2)
    rows = [i for i in want if i < 2048]
    r.manager.allocate("w", tokens[:2048])
    got = r.step([StepEntry("w", tokens[:2048], rows)]).cpu().numpy()
    err = np.array([worst(got[j], want[i]) for j, i in enumerate(rows)])
    assert err.max() <= tol, f"whole prompt: first wrong position {rows[int(np.argmax(err > tol))]} (error {err.max():.3g}, tolerance {tol:.3g})"
    for pos in range(2048, 2048 + 6):
        r.manager.append_slots("w", tokens[pos : pos + 1])
        out = r.step([StepEntry("w", tokens[pos : pos + 1], [0])]).cpu().numpy()
        assert worst(out[0], want[pos]) <= tol, f"decoding at position {pos}: error {worst(out[0], want[pos]):.3g}"
    assert r.graph_steps == 6 and any(key[0] == 1 and set(key[2]) == {16} for key in r.graphs.graphs), sorted(r.graphs.graphs)
    # teeth: the first and the last (half-filled) page of the table change places
    with pages_swapped_in_table(r.manager, "w", 0, (2048 + 6) // 16):
        r.manager.append_slots("w", tokens[2054:2055])
        out = r.step([StepEntry("w", tokens[2054:2055], [0])]).cpu().numpy()
    assert worst(out[0], want[2054]) > tol, "two pages of the table changed places and the logits did not notice"
    r.manager.free("w")
    # the same for the prompt itself, in the second layer only
    r.manager.allocate("m", tokens[:2048])
    with pages_swapped_in_one_layer(r.pools.layer_caches[1], 0, 3, 100):
        got = r.step([StepEntry("m", tokens[:2048], rows)]).cpu().numpy()
    assert max(worst(got[j], want[i]) for j, i in enumerate(rows)) > tol, "two pages changed places in one layer and the logits did not notice"
    assert ops.device_wait_errors() == {}


@pytest.mark.parametrize("num_seqs", [8, 64])
def test_many_sequences_decode_behind_prompts_of_about_2048_tokens(long_1b, num_seqs):
    """8 sequences (graph of 8 rows, eight key splits, the engine's own products with their fused epilogues) and
    64 (graph of 64 rows with none padded, no splits, library products with separate rotary / SiLU / norm
    kernels) decode together behind prompts that are the same tokens cut at different lengths, so every row
    has its own context and its own row of the plain implementation's logits."""
    cfg, path, tokens, want, tol = long_1b
    model = dli_b200.load_model(path, "bfloat16")
    r = runner_with_used_pages(model, num_pages=num_seqs * ((2048 + 32) // 16 + 1), page_size=16, max_requests=num_seqs)
    lens = {f"s{i}": 2048 - (i * 61) % 88 for i in range(num_seqs)}  # 1,961 .. 2,048: pages filled to every degree
    ids = list(lens)
    for at in range(0, num_seqs, 8):  # eight prompts to a step
        for rid in ids[at : at + 8]:
            r.manager.allocate(rid, tokens[: lens[rid]])
        r.step([StepEntry(rid, tokens[: lens[rid]], []) for rid in ids[at : at + 8]])
    for step in range(3):
        for rid in ids:
            r.manager.append_slots(rid, tokens[lens[rid] + step : lens[rid] + step + 1])
        out = r.step([StepEntry(rid, tokens[lens[rid] + step : lens[rid] + step + 1], [0]) for rid in ids]).cpu().numpy()
        err = np.array([worst(out[j], want[lens[rid] + step]) for j, rid in enumerate(ids)])
        assert err.max() <= tol, f"step {step}: sequence {ids[int(np.argmax(err))]} is wrong (error {err.max():.3g}, tolerance {tol:.3g})"
    splits = 8 if num_seqs == 8 else 1
    assert r.graph_steps == 3 and any(key[0] == num_seqs and set(key[2]) == {splits} for key in r.graphs.graphs), sorted(r.graphs.graphs)
    # teeth: in one sequence's table the second page and the last one (half filled: junk behind its tokens) change places
    v = next(j for j, rid in enumerate(ids) if 2 <= (lens[rid] + 4) % 16 <= 12)
    with pages_swapped_in_table(r.manager, ids[v], 1, (lens[ids[v]] + 3) // 16):
        for rid in ids:
            r.manager.append_slots(rid, tokens[lens[rid] + 3 : lens[rid] + 4])
        out = r.step([StepEntry(rid, tokens[lens[rid] + 3 : lens[rid] + 4], [0]) for rid in ids]).cpu().numpy()
    err = np.array([worst(out[j], want[lens[rid] + 3]) for j, rid in enumerate(ids)])
    assert err[v] > tol, "two pages of one sequence's table changed places and its logits did not notice"
    assert np.delete(err, v).max() <= tol, "the other sequences are not touched by it"
    assert ops.device_wait_errors() == {}


def test_one_sequence_decodes_with_more_splits_than_a_cluster_through_the_merge_kernel(tmp_path_factory, monkeypatch):
    """More key splits than one cluster merges (the engine's own policy stays with a cluster; here it is made to ask
    for 24): partial results go to scratch and the merge kernel finishes them; the
    graph's tables are 256 pages wide.  A prompt of 3,100 tokens in two portions, then three tokens decoded."""
    monkeypatch.setattr(attn_kernels, "decode_splits", lambda *sizes: 24)
    cfg, path, weights = model_folder("llama_1b", tmp_path_factory)
    tokens = random_tokens(cfg["vocab_size"], 3100 + 4, seed=14)
    rows = sorted(set(range(2040, 3100, 53)) | set(range(3096, 3104)))
    want = dict(zip(rows, plain.forward(cfg, plain_weights_for(weights, "bfloat16"), tokens, rows=rows, bf16_activations=True)))
    tol = 5e-2 * max(1.0, max(float(np.abs(v).max()) for v in want.values()))
    model = dli_b200.load_model(path, "bfloat16")
    r = runner_with_used_pages(model, num_pages=3200 // 16 + 2, page_size=16, max_requests=2)
    r.manager.allocate("p", tokens[:3100])
    r.step([StepEntry("p", tokens[:2048], [])])
    here = [i for i in rows if 2048 <= i < 3100]
    got = r.step([StepEntry("p", tokens[2048:3100], [i - 2048 for i in here])]).cpu().numpy()
    err = np.array([worst(got[j], want[i]) for j, i in enumerate(here)])
    assert err.max() <= tol, f"second portion: first wrong position {here[int(np.argmax(err > tol))]} (error {err.max():.3g}, tolerance {tol:.3g})"
    for pos in range(3100, 3103):
        r.manager.append_slots("p", tokens[pos : pos + 1])
        out = r.step([StepEntry("p", tokens[pos : pos + 1], [0])]).cpu().numpy()
        assert worst(out[0], want[pos]) <= tol, f"decoding at position {pos}: error {worst(out[0], want[pos]):.3g}"
    assert any(key[0] == 1 and key[1] == 256 and min(key[2]) > 16 for key in r.graphs.graphs), sorted(r.graphs.graphs)
    with pages_swapped_in_table(r.manager, "p", 2, 3103 // 16):  # teeth: the third page and the last, half-filled one
        r.manager.append_slots("p", tokens[3103:3104])
        out = r.step([StepEntry("p", tokens[3103:3104], [0])]).cpu().numpy()
    assert worst(out[0], want[3103]) > tol, "two pages of the table changed places and the logits did not notice"
    assert ops.device_wait_errors() == {}


def test_a_context_of_8000_tokens_at_head_size_128_in_portions_of_2048(tmp_path_factory):
    """The Llama-3.2-3B layer sizes (24 heads on 8, head size 128): a prompt of 8,000 tokens prefilled in portions
    of 2,048, then decoded on from 8,000 (sixteen key splits, merged in a cluster)."""
    cfg, path, weights = model_folder("llama_3b", tmp_path_factory)
    tokens = random_tokens(cfg["vocab_size"], 8000 + 4, seed=12)
    rows = sorted(set(range(5, 8000, 41)) | set(range(7990, 8004)))
    want = dict(zip(rows, plain.forward(cfg, plain_weights_for(weights, "bfloat16"), tokens, rows=rows, bf16_activations=True)))
    tol = 5e-2 * max(1.0, max(float(np.abs(v).max()) for v in want.values()))
    model = dli_b200.load_model(path, "bfloat16")
    r = runner_with_used_pages(model, num_pages=8064 // 16 + 2, page_size=16, max_requests=2)
    r.manager.allocate("p", tokens[:8000])
    for at in range(0, 8000, 2048):
        n = min(2048, 8000 - at)
        here = [i - at for i in rows if at <= i < at + n]
        got = r.step([StepEntry("p", tokens[at : at + n], here)]).cpu().numpy()
        err = np.array([worst(got[j], want[at + i]) for j, i in enumerate(here)])
        assert err.max() <= tol, f"portion at {at}: first wrong position {at + here[int(np.argmax(err > tol))]} (error {err.max():.3g}, tolerance {tol:.3g})"
    for pos in range(8000, 8003):
        r.manager.append_slots("p", tokens[pos : pos + 1])
        out = r.step([StepEntry("p", tokens[pos : pos + 1], [0])]).cpu().numpy()
        assert worst(out[0], want[pos]) <= tol, f"decoding at position {pos}: error {worst(out[0], want[pos]):.3g}"
    assert any(key[0] == 1 and key[2] == (16,) for key in r.graphs.graphs), sorted(r.graphs.graphs)
    # teeth, decoding: the first page and the last one (four tokens, junk behind them) change places in the table
    with pages_swapped_in_table(r.manager, "p", 0, 500):
        r.manager.append_slots("p", tokens[8003:8004])
        out = r.step([StepEntry("p", tokens[8003:8004], [0])]).cpu().numpy()
    assert worst(out[0], want[8003]) > tol, "two pages of the table changed places and the logits did not notice"
    r.manager.free("p")
    # teeth, prompt: the first portion again, two of its pages exchanged in the layer's attention
    r.manager.allocate("m", tokens[:2048])
    here = [i for i in rows if i < 2048]
    with pages_swapped_in_one_layer(r.pools.layer_caches[0], 0, 3, 100):
        got = r.step([StepEntry("m", tokens[:2048], here)]).cpu().numpy()
    assert max(worst(got[j], want[i]) for j, i in enumerate(here)) > tol, "two pages changed places and the logits did not notice"
    assert ops.device_wait_errors() == {}


def test_a_prefix_hit_in_bfloat16_leaves_the_logits_as_they_are(long_1b):
    """Prefix index on, at the benchmark's head size: a second request that begins with 1,000 tokens of the first
    (then goes its own way) finds 992 of them in pages, computes the rest, and decodes; its logits are those
    of the plain implementation run on its own tokens from the start."""
    cfg, path, tokens, want, tol = long_1b
    _, _, weights = _FOLDERS["llama_1b"]
    other = tokens[:1000] + random_tokens(cfg["vocab_size"], 240, seed=13)
    rows = list(range(1000, 1240, 7)) + [1239]
    ref = dict(zip(rows, plain.forward(cfg, plain_weights_for(weights, "bfloat16"), other, rows=rows, bf16_activations=True)))
    model = dli_b200.load_model(path, "bfloat16")
    r = runner_with_used_pages(model, num_pages=2 * (2048 // 16) + 8, page_size=16, max_requests=2, enable_prefix_caching=True)
    r.manager.allocate("first", tokens[:2048])
    r.step([StepEntry("first", tokens[:2048], [])])
    alloc = r.manager.allocate("second", other[:1236])
    assert alloc.num_cached_tokens == 992
    here = [i for i in rows if i < 1236]
    got = r.step([StepEntry("second", other[992:1236], [i - 992 for i in here])]).cpu().numpy()
    err = np.array([worst(got[j], ref[i]) for j, i in enumerate(here)])
    assert err.max() <= tol, f"behind the hit: first wrong position {here[int(np.argmax(err > tol))]} (error {err.max():.3g}, tolerance {tol:.3g})"
    for pos in range(1236, 1240):
        r.manager.append_slots("second", other[pos : pos + 1])
        out = r.step([StepEntry("second", other[pos : pos + 1], [0])]).cpu().numpy()
        if pos in ref:
            assert worst(out[0], ref[pos]) <= tol
    # teeth: the same request once more; in the second layer its first (shared) page and its last one, which holds
    # four of its tokens and junk behind them, change places
    # (from an index that knows the first request only: everything is given back and forgotten, the first runs again)
    r.manager.free("second")
    r.manager.free("first")
    r.manager.reset_prefix_cache()
    r.manager.allocate("first", tokens[:2048])
    r.step([StepEntry("first", tokens[:2048], [])])
    assert r.manager.allocate("again", other[:1236]).num_cached_tokens == 992
    with pages_swapped_in_one_layer(r.pools.layer_caches[1], 0, 0, 77):
        got = r.step([StepEntry("again", other[992:1236], [i - 992 for i in here])]).cpu().numpy()
    assert max(worst(got[j], ref[i]) for j, i in enumerate(here)) > tol, "two pages changed places in one layer and the logits did not notice"
    r.manager.check_invariants()
