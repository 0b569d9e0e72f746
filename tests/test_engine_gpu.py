"""The engine end to end on the GPU: greedy generation through the Python entry point and the
command line against the plain implementation, under a roomy pool, a tiny token budget and a
pool so small that requests are preempted; prefix reuse; seeded sampling that does not depend
on the batch; long decoding; the first tokens of a sequence."""

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import dli_b200
from dli_b200 import LLMEngine, SamplingParams, SchedulerConfig
from dli_b200.engine import FinishReason, ModelRunner, StepEntry
from tests.plain import llama_plain as plain
from tests.util import ROOT, TOL, make_model_dir, plain_weights_for, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in ("tiny_a", "tiny_b"):
        path = tmp_path_factory.mktemp(name)
        cfg, weights, page = make_model_dir(path, name, sharpen=6.0)
        out[name] = (path, cfg, weights, page)
    return out


def plain_greedy_with_margin(cfg, w, prompt, n):
    """Greedy tokens and, for each, the gap between the two largest logits."""
    toks, out, gaps = list(prompt), [], []
    for _ in range(n):
        row = plain.forward(cfg, w, toks)[-1]
        top = np.sort(row)[-2:]
        out.append(int(np.argmax(row)))
        gaps.append(float(top[1] - top[0]))
        toks.append(out[-1])
    return out, gaps


def assert_same_tokens(got, want, gaps, tol, what):
    """Equal up to the first position where the plain top-2 gap is within the tolerance
    (there another rounding may pick the other token, and the sequences part ways)."""
    for i, (g, w_, gap) in enumerate(zip(got, want, gaps)):
        if g != w_:
            assert gap < 2 * tol, f"{what}: token {i} is {g}, plain says {w_} with a gap of {gap:.3g}"
            return
    assert len(got) == len(want)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("setting", ["roomy", "tiny_budget", "tiny_pool"])
def test_greedy_generation_equals_plain(models, name, dtype, setting):
    path, cfg, weights, page = models[name]
    w = plain_weights_for(weights, dtype)
    lens = [5, 17, 33] if name == "tiny_a" else [1, 7, 40, 64, 90]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=n) for n in lens]
    steps = 16
    kwargs = dict(num_blocks=400, config=SchedulerConfig(8, 512))
    if setting == "tiny_budget":
        kwargs = dict(num_blocks=400, config=SchedulerConfig(8, 16))
    if setting == "tiny_pool":
        need = -(-(max(lens) + steps) // page)
        kwargs = dict(num_blocks=need + 3, config=SchedulerConfig(8, 64), watermark=0.0)
    eng = LLMEngine.from_model_dir(path, dtype=dtype, block_size=page, **kwargs)
    outs = eng.generate(prompts, SamplingParams(max_tokens=steps))
    if setting == "tiny_pool":
        assert sum(s.num_preempted for s in eng.stats.steps) > 0, "the pool was not small enough to preempt anybody"
    if setting == "tiny_budget":
        assert max(s.num_batched_tokens for s in eng.stats.steps) <= 16
    for p, got in zip(prompts, outs):
        want, gaps = plain_greedy_with_margin(cfg, w, p, steps)
        assert_same_tokens(got, want, gaps, TOL[dtype], f"{name} {dtype} {setting} prompt of {len(p)}")
    eng.manager.check_invariants()
    assert eng.manager.min_available_pages() == kwargs["num_blocks"]
    # most decode steps were launched before the ids of the step before had been read; an engine
    # that reads first produces the same tokens
    assert eng.lookahead and eng.steps_ahead >= steps // 2
    if setting == "roomy":
        plain_eng = LLMEngine.from_model_dir(path, dtype=dtype, block_size=page, lookahead=False, **kwargs)
        assert plain_eng.generate(prompts, SamplingParams(max_tokens=steps)) == outs and plain_eng.steps_ahead == 0


def test_shared_prefix_is_reused_and_changes_nothing(models):
    path, cfg, weights, page = models["tiny_b"]
    stem = random_tokens(1000, 32, seed=99)
    prompts = [stem + random_tokens(1000, 9, seed=1), stem + random_tokens(1000, 20, seed=2)]
    eng = LLMEngine.from_model_dir(path, dtype="float32", block_size=16, num_blocks=64)
    first = eng.generate(prompts[:1], SamplingParams(max_tokens=8))
    second = eng.generate(prompts[1:], SamplingParams(max_tokens=8))
    assert eng.manager.stats.prompt_tokens_hit == 32
    cold = LLMEngine.from_model_dir(path, dtype="float32", block_size=16, num_blocks=64, enable_prefix_caching=False)
    assert cold.generate(prompts, SamplingParams(max_tokens=8)) == first + second
    assert cold.manager.stats.prompt_tokens_hit == 0


def test_seeded_sampling_alone_busy_and_across_preemption(models):
    """Temperature 0.8 with per-request seeds: a request's tokens are the same alone, in a busy
    batch, and when it is preempted and recomputed (float32, so the logits agree closely)."""
    path, cfg, weights, page = models["tiny_b"]
    prompts = [random_tokens(1000, n, seed=n) for n in (7, 40, 64, 21)]
    params = [SamplingParams(max_tokens=12, temperature=0.8, seed=100 + i, top_k=50 if i % 2 else -1, top_p=0.9 if i > 1 else 1.0) for i in range(4)]
    alone = []
    for p, sp in zip(prompts, params):
        eng = LLMEngine.from_model_dir(path, dtype="float32", block_size=16, num_blocks=64)
        alone.append(eng.generate([p], sp)[0])
    busy = LLMEngine.from_model_dir(path, dtype="float32", block_size=16, num_blocks=64).generate(prompts, params)
    assert busy == alone
    assert LLMEngine.from_model_dir(path, dtype="float32", block_size=16, num_blocks=64, lookahead=False).generate(prompts, params) == alone
    tight = LLMEngine.from_model_dir(path, dtype="float32", block_size=16, num_blocks=8, watermark=0.0)
    assert tight.generate(prompts, params) == alone
    assert sum(s.num_preempted for s in tight.stats.steps) > 0
    # and they are what the plain sampler draws from the plain logits
    toks = list(prompts[1])
    for i, t in enumerate(alone[1][:4]):
        row = plain.forward(cfg, weights, toks)[-1]
        assert t == plain.sample_token(row, 0.8, params[1].top_k, params[1].top_p, 101, i)
        toks.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(models, dtype):
    """One request decoded token by token from its very first token for 300 steps (the logits
    of positions 0, 1, 2 .. are the first tokens of a sequence), against the plain logits."""
    path, cfg, weights, page = models["tiny_b"]
    model = dli_b200.load_model(path, dtype)
    toks = random_tokens(1000, 300, seed=5)
    want = plain.forward(cfg, plain_weights_for(weights, dtype), toks)
    r = ModelRunner(model, num_pages=20, page_size=16, enable_prefix_caching=False, watermark=0.0)
    got = []
    for i, t in enumerate(toks):
        if i == 0:
            r.manager.allocate("x", [t])
        else:
            r.manager.append_slots("x", [t])
        got.append(r.step([StepEntry("x", [t], [0])]))
    got = torch.cat(got).cpu().numpy()
    err = np.abs(got - want).max(axis=1)
    bad = np.nonzero(err > TOL[dtype])[0]
    assert bad.size == 0, f"first wrong position {bad[0]} (error {err[bad[0]]:.3g})"


def test_stop_reasons_and_capacity(models):
    path, cfg, weights, page = models["tiny_a"]
    eng = LLMEngine.from_model_dir(path, dtype="float32", block_size=4, num_blocks=10)
    prompt = random_tokens(256, 6, seed=1)
    free_run = eng.generate([prompt], SamplingParams(max_tokens=10))[0]
    stop = eng.add_request("s", prompt, SamplingParams(max_tokens=10, stop_token_ids=(free_run[3],)))
    big = eng.add_request("b", prompt, SamplingParams(max_tokens=40))
    while eng.has_unfinished():
        eng.step()
    assert stop.output_ids == free_run[: free_run.index(free_run[3]) + 1] and stop.finish_reason is FinishReason.STOP
    assert big.finish_reason is FinishReason.CAPACITY and big.output_ids == []
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.generate([[300]], SamplingParams(max_tokens=1))


def test_command_line_generates(models, tmp_path):
    path, cfg, weights, page = models["tiny_a"]
    prompt = random_tokens(256, 9, seed=3)
    cmd = [sys.executable, str(ROOT / "bin" / "dli"), "generate", "--model", str(path), "--dtype", "float32", "--block-size", "4",
           "--num-blocks", "64", "--max-num-batched-tokens", "8", "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--ignore-eos"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    want, gaps = plain_greedy_with_margin(cfg, weights, prompt, 6)
    assert_same_tokens(rec["output_ids"], want, gaps, TOL["float32"], "cli")
    assert rec["finish_reason"] == "length"
    # and `dli init` writes a folder the engine loads
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "dli"), "init", "--config", str(tmp_path / "c.json"), "--seed", "0", "--out", str(tmp_path / "m")],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert (tmp_path / "m" / "model.safetensors").exists()
    # and `dli bench` times decode steps of a batch on random weights
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "dli"), "bench", "--random-config", str(tmp_path / "c.json"), "--batch", "3",
                          "--input-len", "20", "--output-len", "40", "--steps", "5", "--warmup", "2", "--block-size", "8"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["batch"] == 3 and rec["tokens_per_s"] > 0 and rec["steps_launched_ahead"] >= 5 and rec["bandwidth_floor_ms"] > 0
    # and `dli workload` runs a closed set of requests, half of them behind a shared prefix, in a pool that makes some wait
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "dli"), "workload", "--random-config", str(tmp_path / "c.json"), "--num-requests", "9",
                          "--min-input", "5", "--max-input", "40", "--output-len", "12", "--shared-prefix-len", "16", "--shared-fraction", "0.6",
                          "--block-size", "4", "--max-num-seqs", "4", "--max-num-batched-tokens", "24", "--num-blocks", "40"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["requests"] == 9 and rec["generated_tokens"] == 9 * 12 and rec["prompt_tokens_reused"] > 0
    assert rec["decode_tokens_run"] >= 9 * 11 and rec["generated_tokens_per_s"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generate_with_and_without_cache(models, dtype):
    """The plain entry point: the cached path, the path that runs the whole sequence again for every
    token, and the plain implementation agree; a stop id ends the generation and is kept."""
    import dli_b200

    path, cfg, weights, page = models["tiny_a"]
    model = dli_b200.load_model(path, dtype)
    prompt = random_tokens(cfg["vocab_size"], 21, seed=5)
    cached = dli_b200.greedy_generate(model, prompt, 12, page_size=page)
    want, gaps = plain_greedy_with_margin(cfg, plain_weights_for(weights, dtype), prompt, 12)
    assert_same_tokens(cached, want, gaps, TOL[dtype], f"greedy_generate {dtype}")
    again = dli_b200.greedy_generate(model, prompt, 12, use_cache=False, page_size=page)
    assert_same_tokens(again, want, gaps, TOL[dtype], f"greedy_generate without cache {dtype}")
    assert dli_b200.greedy_generate(model, prompt, 12, eos_token_ids=[cached[3]], page_size=page) == cached[: cached.index(cached[3]) + 1]
    assert dli_b200.greedy_generate(model, prompt, 0) == []
    with pytest.raises(ValueError):
        dli_b200.greedy_generate(model, [], 3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forked_requests_continue_apart(models, dtype):
    """Two continuations of one prompt share its pages; the first append into the shared, partly
    filled last page copies it (all layers), after which each request's logits are those of its own
    sequence, in one batch and step by step."""
    path, cfg, weights, page = models["tiny_b"]
    w = plain_weights_for(weights, dtype)
    model = dli_b200.load_model(path, dtype)
    runner = ModelRunner(model, num_pages=16, page_size=page, max_requests=4, enable_prefix_caching=False, watermark=0.0)
    prompt = random_tokens(cfg["vocab_size"], page + page // 2 + 1, seed=9)  # ends inside its second page
    runner.manager.allocate("a", prompt)
    runner.step([StepEntry("a", prompt, [len(prompt) - 1])])
    runner.manager.fork("a", "b")
    seqs = {"a": list(prompt), "b": list(prompt)}
    for step in range(page):  # long enough to leave the copied page and open a new one
        entries = []
        for rid in ("a", "b"):
            tok = (7 + 3 * step) % cfg["vocab_size"] if rid == "a" else (11 + 5 * step) % cfg["vocab_size"]
            copies = runner.manager.append_slots(rid, [tok])
            assert bool(copies) == (step == 0 and rid == "a"), "exactly the first appender gets a page of its own"
            runner.copy_pages(copies)
            seqs[rid].append(tok)
            entries.append(StepEntry(rid, [tok], [0]))
        got = runner.step(entries).float().cpu().numpy()
        for row, rid in enumerate(("a", "b")):
            want = plain.forward(cfg, w, seqs[rid])[-1]
            np.testing.assert_allclose(got[row], want, atol=TOL[dtype], err_msg=f"{rid} step {step}")
    runner.manager.check_invariants()
    runner.manager.free("a"), runner.manager.free("b")
    assert runner.manager.min_available_pages() == 16
