"""Small steps that mix prompt portions with decoded tokens, replayed from captured graphs: their logits, and the
cache they leave, against the same steps launched kernel by kernel and against the plain implementation."""

import numpy as np
import pytest
import torch

import dli_b200
from dli_b200.engine import ModelRunner, StepEntry
from tests.plain import llama_plain as plain
from tests.test_real_shapes_gpu import model_folder
from tests.util import TOL, make_model_dir, plain_weights_for, random_tokens

pytestmark = pytest.mark.gpu


def runner_for(model, page, graphs: bool):
    r = ModelRunner(model, num_pages=400, page_size=page, max_requests=16, enable_prefix_caching=False, watermark=0.0, cuda_graphs=graphs)
    if graphs:
        r.graphs.mixed_after = 1  # capture a shape when it first comes
    return r


def run_schedule(runner, prompts, schedule):
    """``schedule``: steps of [(request, tokens to bring, wanted places)]; returns each step's logits."""
    done = {i: 0 for i in prompts}
    out = []
    for step in schedule:
        entries = []
        for rid, count, want in step:
            if done[rid] == 0:
                runner.manager.allocate(rid, prompts[rid])
                runner.start_request(rid, runner.manager.state_slot(rid))
            entries.append(StepEntry(rid, prompts[rid][done[rid] : done[rid] + count], want))
            done[rid] += count
        out.append(runner.step(entries).float().cpu().numpy())
    for rid in prompts:
        if done[rid]:
            runner.manager.free(rid)
    runner.manager.check_invariants()
    return out


# requests 0-2 decode token by token after a first whole step; 3-5 arrive in portions beside them
SCHEDULE = [
    [(0, 20, [19]), (1, 33, [32]), (2, 5, [4])],               # three prompts whole (three portions, no single token)
    [(0, 1, [0]), (1, 1, [0]), (2, 1, [0]), (3, 17, [])],       # three decoded tokens beside a portion that wants nothing
    [(3, 9, [8]), (0, 1, [0]), (1, 1, [0]), (2, 1, [0])],       # the portion first in the caller's order; it ends here
    [(0, 1, [0]), (4, 30, [0, 29]), (5, 2, [1]), (1, 1, [])],   # two portions, one of two tokens; two places of one portion
    [(4, 3, [2]), (5, 21, [20]), (3, 1, [0]), (0, 1, [0]), (1, 1, [0]), (2, 1, [0])],
    [(0, 1, [0]), (1, 1, [0]), (2, 1, [0]), (3, 1, [0]), (4, 1, [0]), (5, 1, [0])],  # all decode: the cache the graphs left
]


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_steps_from_graphs_equal_the_same_steps_launched_one_by_one(tmp_path, name, dtype):
    cfg, weights, page = make_model_dir(tmp_path, name, sharpen=6.0)
    w = plain_weights_for(weights, dtype)
    model = dli_b200.load_model(tmp_path, dtype=dtype)
    vocab = cfg["vocab_size"]
    prompts = {i: random_tokens(vocab, 64, 100 + i) for i in range(6)}
    with_graphs, eager = runner_for(model, page, True), runner_for(model, page, False)
    got, want = run_schedule(with_graphs, prompts, SCHEDULE), run_schedule(eager, prompts, SCHEDULE)
    assert with_graphs.mixed_graph_steps == len(SCHEDULE) - 1 and with_graphs.graph_steps == 1 and len(with_graphs.graphs.mixed) >= 2, (
        with_graphs.mixed_graph_steps, with_graphs.graphs.mixed_failure)
    for step, (a, b) in enumerate(zip(got, want)):
        assert a.shape == b.shape, step
        np.testing.assert_allclose(a, b, atol=TOL[dtype], err_msg=f"step {step}")
    # and against the plain implementation: the last step's logits of every request
    done = {i: 0 for i in prompts}
    for step in SCHEDULE:
        for rid, count, _ in step:
            done[rid] += count
    for row, rid in enumerate(range(6)):
        ref = plain.forward(cfg, w, prompts[rid][: done[rid]])[-1]
        np.testing.assert_allclose(got[-1][row], ref, atol=TOL[dtype], err_msg=f"request {rid}")
    # the same shapes again replay the graphs that exist
    before = len(with_graphs.graphs.mixed)
    again = run_schedule(with_graphs, {i: random_tokens(vocab, 64, 200 + i) for i in range(6)}, SCHEDULE)
    assert len(with_graphs.graphs.mixed) == before and len(again) == len(SCHEDULE)


def test_a_shape_is_captured_once_it_has_come_often_enough(tmp_path):
    cfg, _, page = make_model_dir(tmp_path, "tiny_a")
    model = dli_b200.load_model(tmp_path, dtype="bfloat16")
    r = ModelRunner(model, num_pages=500, page_size=page, max_requests=4, enable_prefix_caching=False, watermark=0.0)
    assert r.graphs.mixed_after >= 8  # a capture costs many steps: by default only shapes that keep coming
    r.graphs.mixed_after = 2
    toks = random_tokens(cfg["vocab_size"], 40, 1)
    for i in range(3):
        r.manager.allocate(i, toks[: 20 + i])  # 20, 21, 22 tokens: one bucket
        r.step([StepEntry(i, toks[: 20 + i], [19 + i])])
        assert (len(r.graphs.mixed), r.mixed_graph_steps) == [(0, 0), (1, 1), (1, 2)][i]
        r.manager.free(i)
    r.manager.allocate("long", toks * 40)  # 1,600 tokens: past the buckets, launched kernel by kernel
    r.step([StepEntry("long", toks * 40, [1599])])
    assert (len(r.graphs.mixed), r.mixed_graph_steps) == (1, 2)


def test_mixed_graphs_at_the_benchmark_sizes(tmp_path_factory):
    """Llama-3.2-1B layer sizes (two layers): 7 decoding sequences at contexts around 300 beside a portion of 200
    tokens, then a step with two portions; tensor-core attention, the library's products at these token counts."""
    cfg, path, weights = model_folder("llama_1b", tmp_path_factory)
    w = plain_weights_for(weights, "bfloat16")
    model = dli_b200.load_model(path, dtype="bfloat16")
    vocab = cfg["vocab_size"]
    prompts = {i: random_tokens(vocab, 600, 300 + i) for i in range(10)}
    first = [(i, 290 + 3 * i, [289 + 3 * i]) for i in range(7)]
    schedule = [
        first,                                                            # 7 prompts: more than the graphs' four portions
        [(i, 1, [0]) for i in range(7)] + [(7, 200, [199])],
        [(7, 130, [129])] + [(i, 1, [0]) for i in range(7)] + [(8, 70, [])],
        [(i, 1, [0]) for i in range(9)],
    ]
    with_graphs = ModelRunner(model, num_pages=500, page_size=16, max_requests=16, enable_prefix_caching=False, watermark=0.0)
    with_graphs.graphs.mixed_after = 1
    eager = ModelRunner(model, num_pages=500, page_size=16, max_requests=16, enable_prefix_caching=False, watermark=0.0, cuda_graphs=False)
    got, want = run_schedule(with_graphs, prompts, schedule), run_schedule(eager, prompts, schedule)
    assert with_graphs.mixed_graph_steps == 2 and with_graphs.graph_steps == 1 and len(with_graphs.graphs.mixed) == 1
    scale = float(np.abs(want[-1]).max())
    for step, (a, b) in enumerate(zip(got, want)):
        np.testing.assert_allclose(a, b, atol=0.02 * scale, err_msg=f"step {step}")
    # against the plain implementation, rounded where a bfloat16 model rounds, with the tolerance of the other tests at these sizes
    ref = plain.forward(cfg, w, prompts[7][:331], rows=[330], bf16_activations=True)[0]
    np.testing.assert_allclose(got[-1][7], ref, atol=5e-2 * max(1.0, float(np.abs(ref).max())))
