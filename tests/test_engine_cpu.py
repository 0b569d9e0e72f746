"""The engine's host side end to end on the CPU: the real parts, cache pools, step function, scheduler
and LLMEngine in float32, with torch stand-ins for the kernels (tests/cpu_ops.py), against the plain
implementation.  The GPU tests make the same comparisons with the real kernels."""

import sys

import numpy as np
import pytest
import torch

import dli_b200
from dli_b200 import LLMEngine, SamplingParams, SchedulerConfig
from dli_b200.engine import ModelRunner, PagedSequence, StepEntry, paged_greedy_generate
from tests import cpu_ops
from tests.plain import llama_plain as plain
from tests.util import make_model_dir, plain_weights_for, random_tokens

TOL = 2e-4
TOLS = {"float32": 2e-4, "bfloat16": 5e-2}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in ("tiny_a", "tiny_b", "tiny_c"):
        path = tmp_path_factory.mktemp(name)
        cfg, weights, page = make_model_dir(path, name, sharpen=6.0)
        out[name] = (path, cfg, weights, page)
    return out


@pytest.fixture(autouse=True)
def cpu_kernels():
    with cpu_ops.patched():
        yield


def engine_for(path, page, num_blocks, config=None, dtype="float32", **kw):
    model = dli_b200.load_model(path, dtype, "cpu")
    config = config or SchedulerConfig(8, 512)
    runner = ModelRunner(model, num_pages=num_blocks, page_size=page, max_requests=config.max_num_seqs, cuda_graphs=False,
                         enable_prefix_caching=kw.pop("enable_prefix_caching", True), watermark=kw.pop("watermark", 0.01))
    return LLMEngine(runner, config, sampler=cpu_ops.CpuSampler(), **kw)


def plain_greedy(cfg, w, prompt, n):
    toks, out, gaps = list(prompt), [], []
    for _ in range(n):
        row = plain.forward(cfg, w, toks)[-1]
        top = np.sort(row)[-2:]
        out.append(int(np.argmax(row)))
        gaps.append(float(top[1] - top[0]))
        toks.append(out[-1])
    return out, gaps


def same_tokens(got, want, gaps, what, tol=TOL):
    for i, (g, w_, gap) in enumerate(zip(got, want, gaps)):
        if g != w_:
            assert gap < 2 * tol, f"{what}: token {i} is {g}, plain says {w_} with a gap of {gap:.3g}"
            return
    assert len(got) == len(want)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
def test_whole_prompt_logits_equal_plain(models, name):
    path, cfg, weights, page = models[name]
    model = dli_b200.load_model(path, "float32", "cpu")
    toks = random_tokens(cfg["vocab_size"], 37, seed=4)
    runner = ModelRunner(model, num_pages=12, page_size=page, cuda_graphs=False, enable_prefix_caching=False, watermark=0.0)
    runner.manager.allocate("x", toks)
    got = runner.step([StepEntry("x", toks, list(range(len(toks))))]).numpy()
    np.testing.assert_allclose(got, plain.forward(cfg, weights, toks), atol=TOL)
    # portions of changing size, down to two tokens, and then token by token: the same logits
    runner.manager.free("x")
    runner.manager.allocate("y", toks[:30])
    rows, at = [], 0
    for n in (7, 2, 16, 3, 2):
        rows.append(runner.step([StepEntry("y", toks[at : at + n], list(range(n)))]))
        at += n
    for t in toks[30:]:
        runner.manager.append_slots("y", [t])
        rows.append(runner.step([StepEntry("y", [t], [0])]))
    np.testing.assert_allclose(torch.cat(rows).numpy(), got, atol=TOL)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
@pytest.mark.parametrize("setting", ["roomy", "tiny_budget", "tiny_pool"])
@pytest.mark.parametrize("lookahead", [True, False])
def test_greedy_generation_equals_plain(models, name, setting, lookahead):
    path, cfg, weights, page = models[name]
    lens = [5, 17, 33] if name == "tiny_a" else [1, 7, 40]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=n) for n in lens]
    steps = 10
    kwargs = dict(num_blocks=200, config=SchedulerConfig(8, 512))
    if setting == "tiny_budget":
        kwargs = dict(num_blocks=200, config=SchedulerConfig(8, 16))
    if setting == "tiny_pool":
        # every prompt is admitted at once and the pool is full then: the first page anybody needs is somebody else's
        blocks = max(-(-(max(lens) + steps) // page), sum(-(-n // page) for n in lens))
        kwargs = dict(num_blocks=blocks, config=SchedulerConfig(8, 64), watermark=0.0)
    eng = engine_for(path, page, lookahead=lookahead, **kwargs)
    assert eng.lookahead == lookahead
    outs = eng.generate(prompts, SamplingParams(max_tokens=steps))
    if setting == "tiny_pool":
        assert sum(s.num_preempted for s in eng.stats.steps) > 0, "the pool was not small enough to preempt anybody"
    if setting == "tiny_budget":
        assert max(s.num_batched_tokens for s in eng.stats.steps) <= 16
    for p, got in zip(prompts, outs):
        want, gaps = plain_greedy(cfg, weights, p, steps)
        same_tokens(got, want, gaps, f"{name} {setting} prompt of {len(p)}")
    eng.manager.check_invariants()
    assert eng.manager.min_available_pages() == kwargs["num_blocks"] and not eng._unknown
    if lookahead:
        assert eng.steps_ahead >= steps // 2


def test_shared_prefix_priorities_and_seeded_sampling(models):
    path, cfg, weights, page = models["tiny_b"]
    stem = random_tokens(1000, 32, seed=99)
    prompts = [stem + random_tokens(1000, 9, seed=1), stem + random_tokens(1000, 20, seed=2), random_tokens(1000, 12, seed=3)]
    params = [SamplingParams(max_tokens=6, temperature=0.8, seed=100 + i, top_k=50 if i % 2 else -1, top_p=0.9 if i > 1 else 1.0) for i in range(3)]
    alone = [engine_for(path, 16, 64).generate([p], sp)[0] for p, sp in zip(prompts, params)]
    eng = engine_for(path, 16, 64, config=SchedulerConfig(2, 24, tenant_weights={"t": 2.0}))
    first = eng.generate(prompts[:1], params[0])
    reqs = [eng.add_request(f"r{i}", p, sp, priority=dli_b200.Priority.BATCH if i == 2 else dli_b200.Priority.INTERACTIVE, tenant="t" if i else "u")
            for i, (p, sp) in enumerate(zip(prompts, params)) if i]
    while eng.has_unfinished():
        eng.step()
    assert [first[0]] + [r.output_ids for r in reqs] == alone  # a request's tokens do not depend on its company or its place in the order
    assert eng.manager.stats.prompt_tokens_hit == 32
    toks = list(prompts[1])
    for i, t in enumerate(alone[1][:3]):  # and they are what the plain sampler draws from the plain logits
        assert t == plain.sample_token(plain.forward(cfg, weights, toks)[-1], 0.8, params[1].top_k, params[1].top_p, 101, i)
        toks.append(t)


def test_paged_sequence_on_the_real_runner(models):
    path, cfg, weights, page = models["tiny_a"]
    model = dli_b200.load_model(path, "float32", "cpu")
    runner = ModelRunner(model, num_pages=40, page_size=page, cuda_graphs=False, watermark=0.0)
    pick = lambda row: int(row.argmax())  # noqa: E731
    stem = random_tokens(256, 13, seed=8)
    a = paged_greedy_generate(runner, "a", stem + [5, 6], 6, pick=pick)
    want, gaps = plain_greedy(cfg, weights, stem + [5, 6], 6)
    same_tokens(a.tokens, want, gaps, "first")
    b = paged_greedy_generate(runner, "b", stem + [7], 4, pick=pick, release=False)
    assert b.num_cached_prompt_tokens == 12
    want, gaps = plain_greedy(cfg, weights, stem + [7], 4)
    same_tokens(b.tokens, want, gaps, "behind the reused pages")
    hist = stem + [7] + b.tokens[:-1]
    row = PagedSequence(runner, "b").feed(9)  # a forced token
    np.testing.assert_allclose(row.numpy(), plain.forward(cfg, weights, hist + [9])[-1], atol=TOL)
    # a fork continues apart from its parent: the shared last page is copied before it is written
    runner.manager.fork("b", "c")
    rb = PagedSequence(runner, "b").feed(11)
    rc = PagedSequence(runner, "c").feed(12)
    np.testing.assert_allclose(rb.numpy(), plain.forward(cfg, weights, hist + [9, 11])[-1], atol=TOL)
    np.testing.assert_allclose(rc.numpy(), plain.forward(cfg, weights, hist + [9, 12])[-1], atol=TOL)
    runner.manager.free("b"), runner.manager.free("c")
    runner.manager.check_invariants()


@pytest.mark.parametrize("how", ["script", "command"])
def test_trace_run_in_process(models, tmp_path, monkeypatch, capsys, how):
    """bin/trace_run itself (its arguments, the order of the wanted rows, requests that end and whose
    pages are used again), run in this process on the stand-ins: up to four live requests, portions of
    some beside single tokens of others, in a pool of 128 tokens."""
    import io
    import json
    import runpy
    import sys

    from tests.util import ROOT

    path, cfg, weights, page = models["tiny_b"]
    seqs = {k: random_tokens(1000, n, seed=40 + i) for i, (k, n) in enumerate((("a", 40), ("b", 23), ("c", 31), ("d", 12), ("e", 50)))}
    full = {k: plain.forward(cfg, weights, v) for k, v in seqs.items()}
    at = dict.fromkeys(seqs, 0)

    def portion(k, n, want):
        toks = seqs[k][at[k] : at[k] + n]
        rows = [at[k] + w for w in want]
        at[k] += n
        return {"id": k, "tokens": toks, "want": want}, [(k, r) for r in rows]

    plan = [  # (entries, end)
        ([("a", 17, [0, 16]), ("b", 23, [22])], []),
        ([("a", 2, [1]), ("c", 16, [])], ["b"]),
        ([("a", 1, [0]), ("c", 15, [14, 0]), ("d", 12, [11])], []),
        ([("a", 20, [19])], ["a", "d", "c"]),
        ([("e", 48, [47])], []),  # needs pages that a, c and d gave back
        ([("e", 1, [0])], []),
        ([("e", 1, [0])], ["e"]),
    ]
    lines, expected = [], []
    for step, (entries, end) in enumerate(plan):
        recs, rows = [], []
        for k, n, want in entries:
            rec, r = portion(k, n, want)
            recs.append(rec)
            rows += r
        lines.append(json.dumps({"step": step, "entries": recs, "end": end}))
        expected.append(rows)
    out_dir = tmp_path / "logits"
    argv = ["--model", str(path), "--dtype", "float32", "--out", str(out_dir), "--max-tokens", "128", "--device", "cpu"]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(lines) + "\n"))
    if how == "script":  # bin/trace_run, as its own program
        monkeypatch.setattr(sys, "argv", ["trace_run", *argv])
        with pytest.raises(SystemExit) as done:
            runpy.run_path(str(ROOT / "bin" / "trace_run"), run_name="__main__")
        assert done.value.code == 0
    else:  # the same through the command line's `dli replay`
        from dli_b200 import cli

        assert cli.main(["replay", *argv]) == 0
    assert capsys.readouterr().out.split() == [w for step in range(len(plan)) for w in ("done", str(step))]
    for step, rows in enumerate(expected):
        got = np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(len(rows), -1)
        want = np.stack([full[k][r] for k, r in rows])
        np.testing.assert_allclose(got, want, atol=TOL, err_msg=f"step {step}")


def test_trace_run_with_the_prefix_index_on(models, tmp_path, monkeypatch, capsys):
    """--prefix-caching: a request whose tokens begin like an earlier one's (ended, or still live) is not run over
    the shared pages again, and its logits are what they are without the index."""
    import io
    import json

    from dli_b200 import replay

    path, cfg, weights, page = models["tiny_b"]  # pages of 16 tokens
    stem = random_tokens(1000, 50, seed=70)
    seqs = {"a": stem + random_tokens(1000, 9, seed=71), "b": stem + random_tokens(1000, 14, seed=72), "c": stem[:40] + random_tokens(1000, 20, seed=73)}
    full = {k: plain.forward(cfg, weights, v) for k, v in seqs.items()}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": seqs["a"], "want": list(range(59))}], "end": ["a"]},
        # b: the stem's three full pages are idle in the index; places 50.. are wanted
        {"step": 1, "entries": [{"id": "b", "tokens": seqs["b"][:60], "want": list(range(50, 60))}], "end": []},
        # c shares two pages with b while b is live; b goes on beside it
        {"step": 2, "entries": [{"id": "c", "tokens": seqs["c"], "want": list(range(40, 60))}, {"id": "b", "tokens": seqs["b"][60:], "want": [0, 3]}], "end": ["b", "c"]},
    ]
    rows = [[("a", i) for i in range(59)], [("b", i) for i in range(50, 60)], [("c", i) for i in range(40, 60)] + [("b", 60), ("b", 63)]]
    out_dir = tmp_path / "logits"
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    assert replay.main(["--model", str(path), "--dtype", "float32", "--out", str(out_dir), "--max-tokens", "192", "--device", "cpu", "--prefix-caching"]) == 0
    err = capsys.readouterr().err
    assert "request b: 48 tokens found" in err and "request c: 32 tokens found" in err
    for step, want_rows in enumerate(rows):
        got = np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(len(want_rows), -1)
        np.testing.assert_allclose(got, np.stack([full[k][r] for k, r in want_rows]), atol=TOL, err_msg=f"step {step}")


# ---- bfloat16: the decode products with their fused epilogues, and the choice of attention kernels


TINY_D64 = {  # head size 64, so that the dispatch takes the TMA-fed decode kernel and the tcgen05 prefill kernel
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192, "vocab_size": 300, "rope_theta": 10000.0,
    "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 256, "hidden_act": "silu",
}


@pytest.fixture(scope="module")
def model_d64(tmp_path_factory):
    import torch as _torch

    from dli_b200.weights import write_safetensors

    path = tmp_path_factory.mktemp("tiny_d64")
    dli_b200.write_model_dir(path, TINY_D64, seed=7)
    w = {k: _torch.from_numpy(v.copy()) for k, v in plain.read_safetensors(path / "model.safetensors").items()}
    for k in w:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            w[k] = w[k] * 6.0
    write_safetensors(path / "model.safetensors", w)
    return path, TINY_D64, plain.read_safetensors(path / "model.safetensors"), 16


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "d64"])
def test_bfloat16_logits_whole_in_portions_and_token_by_token(models, model_d64, name):
    """In bfloat16 a step of up to 8 tokens takes the decode products (rotary and cache write, SiLU * up,
    residual + the first half of the next norm in their epilogues; the norm's factor applied by the product
    that reads the rows); longer portions take the library's products and the separate kernels.  Both, and
    every way of cutting, give the plain logits."""
    path, cfg, weights, page = model_d64 if name == "d64" else models[name]
    w = plain_weights_for(weights, "bfloat16")
    model = dli_b200.load_model(path, "bfloat16", "cpu")
    toks = random_tokens(cfg["vocab_size"], 41, seed=6)
    want = plain.forward(cfg, w, toks)
    runner = ModelRunner(model, num_pages=12, page_size=page, cuda_graphs=False, enable_prefix_caching=False, watermark=0.0)
    runner.manager.allocate("x", toks)
    got = runner.step([StepEntry("x", toks, list(range(len(toks))))]).numpy()
    np.testing.assert_allclose(got, want, atol=TOLS["bfloat16"])
    runner.manager.free("x")
    runner.manager.allocate("y", toks[:30])
    rows, at = [], 0
    for n in (9, 2, 12, 4, 3):  # portions above and below the 8 tokens that the decode products take
        rows.append(runner.step([StepEntry("y", toks[at : at + n], list(range(n)))]))
        at += n
    for t in toks[30:]:
        runner.manager.append_slots("y", [t])
        rows.append(runner.step([StepEntry("y", [t], [0])]))
    np.testing.assert_allclose(torch.cat(rows).numpy(), want, atol=TOLS["bfloat16"])
    # the paths that were meant to run did run
    ran = cpu_ops.calls
    assert ran.get("skinny_gemm_residual", 0) > 0 and ran.get("add_rmsnorm", 0) > 0 and ran.get("silu_mul", 0) > 0
    assert ran.get("skinny_gemm_rotary", 0) > 0 or cfg["head_dim"] == 48  # a head of 48 does not divide the product's tile
    assert (ran.get("skinny_gemm_swiglu", 0) > 0) == (cfg["intermediate_size"] % 64 == 0)
    if name == "d64":
        assert ran.get("paged_decode_tma", 0) > 0 and ran.get("paged_prefill_tc", 0) > 0 and "paged_attention_mma" not in ran
    else:
        assert ran.get("paged_attention_mma", 0) > 0 and "paged_decode_tma" not in ran


@pytest.mark.parametrize("lookahead", [True, False])
def test_bfloat16_generation_mixed_batches(models, lookahead):
    path, cfg, weights, page = models["tiny_a"]
    w = plain_weights_for(weights, "bfloat16")
    prompts = [random_tokens(256, n, seed=n) for n in (5, 17, 33, 2)]
    eng = engine_for(path, page, 200, config=SchedulerConfig(8, 20), dtype="bfloat16", lookahead=lookahead)
    outs = eng.generate(prompts, SamplingParams(max_tokens=8))
    for p, got in zip(prompts, outs):
        want, gaps = plain_greedy(cfg, w, p, 8)
        same_tokens(got, want, gaps, f"prompt of {len(p)}", TOLS["bfloat16"])
    eng.manager.check_invariants()


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
def test_engine_tokens_equal_the_reference_engine_run(name, tmp_path):
    """tests/golden/<name>.npz holds 16 greedy tokens that the reference's own model produced from the first 9
    ids of its sequence, on the weights this repository's writer makes for the configuration's seed.  The engine
    (float32, CPU stand-ins), alone and in a batch with other requests, produces the same tokens."""
    from pathlib import Path

    from tests.tiny_configs import TINY

    cfg, seed, page = TINY[name]
    gold = np.load(Path(__file__).parent / "golden" / f"{name}.npz")
    dli_b200.write_model_dir(tmp_path, cfg, seed)
    prompt = gold["token_ids"][:9].tolist()
    eng = engine_for(tmp_path, page, 64, config=SchedulerConfig(4, 7))
    others = [random_tokens(cfg["vocab_size"], n, seed=n) for n in (3, 20)]
    outs = eng.generate([others[0], prompt, others[1]], SamplingParams(max_tokens=16))
    assert outs[1] == gold["greedy"].tolist()
