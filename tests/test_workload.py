"""The closed-loop runner and the command line around it, with a model that has no tensors (no GPU)."""

import json
import types

import pytest

from dli_b200 import SamplingParams, cli
from dli_b200.engine import LLMEngine, percentile, run_closed_loop
from tests.fake_runner import fake_engine, sequential


@pytest.mark.parametrize("ahead", [False, True])
@pytest.mark.parametrize("concurrency", [None, 1, 3])
def test_closed_loop_keeps_the_concurrency_and_loses_nothing(ahead, concurrency):
    eng, runner = fake_engine(ahead=ahead, max_num_seqs=8, budget=16)
    prompts = [[i, i + 1, i + 2] * (1 + i % 4) for i in range(10)]
    in_flight = []
    step = eng.step

    def counting_step():
        in_flight.append(len(eng.scheduler.running) + len(eng.scheduler.waiting))
        return step()

    eng.step = counting_step
    ticks = iter(range(10**6))
    run = run_closed_loop(eng, prompts, SamplingParams(max_tokens=6), concurrency=concurrency, clock=lambda: float(next(ticks)))
    assert [r.output_ids for r in run.requests] == [sequential(p, 6) for p in prompts]
    assert max(in_flight) <= (concurrency or len(prompts))
    if concurrency:
        assert max(in_flight) == concurrency
    assert len(run.submitted_s) == len(run.first_token_s) == len(run.done_s) == 10 and run.steps == len(in_flight)
    ttft, tpot = run.time_to_first_token(), run.time_per_output_token()
    assert len(ttft) == 10 and len(tpot) == 10 and ttft[0] > 0 and tpot[0] > 0 and run.seconds > 0
    if concurrency == 1:  # one at a time: a request is submitted only after the one before is done
        order = sorted(run.submitted_s, key=run.submitted_s.get)
        assert all(run.done_s[a] <= run.submitted_s[b] for a, b in zip(order, order[1:]))
    eng.manager.check_invariants()
    assert not eng.has_unfinished()


def test_closed_loop_counts_a_refused_request_as_done_and_checks_its_arguments():
    eng, _ = fake_engine(num_pages=4, page_size=4)
    run = run_closed_loop(eng, [[1] * 30, [1, 2]], SamplingParams(max_tokens=3), concurrency=1)
    assert run.requests[0].finish_reason.value == "capacity" and run.requests[1].output_ids == sequential([1, 2], 3)
    assert len(run.time_to_first_token()) == 1
    with pytest.raises(ValueError):
        run_closed_loop(eng, [[1]], SamplingParams(), concurrency=0)
    with pytest.raises(ValueError):
        run_closed_loop(eng, [[1], [2]], [SamplingParams()])


def test_percentile():
    assert percentile([], 0.5) is None and percentile([3.0], 0.99) == 3.0
    assert percentile([1, 2, 3, 4, 5], 0.5) == 3 and percentile([1, 2, 3, 4, 5], 0.99) == 5 and percentile([1, 2, 3, 4, 5], 0.0) == 1


def test_workload_command_with_a_fake_engine(monkeypatch, capsys, tmp_path):
    """The command's own arithmetic and record, around an engine without tensors."""
    import torch

    made = {}

    def for_model(model, *, num_blocks, block_size, config, **kw):
        eng, runner = fake_engine(num_pages=num_blocks, page_size=block_size, max_num_seqs=config.max_num_seqs, budget=config.max_num_batched_tokens)
        runner.graph_steps = runner.mixed_graph_steps = 0
        made["engine"], made["blocks"] = eng, num_blocks
        return eng

    monkeypatch.setattr(cli, "_model_for", lambda args: types.SimpleNamespace(spec=types.SimpleNamespace(vocab_size=50)))
    monkeypatch.setattr(LLMEngine, "for_model", staticmethod(for_model))
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a: None)
    monkeypatch.setattr(torch.cuda, "max_memory_allocated", lambda *a: 0)
    rc = cli.main(["workload", "--random-config", "llama-3.2-1b", "--num-requests", "12", "--min-input", "3", "--max-input", "30",
                   "--output-len", "5", "--shared-prefix-len", "8", "--shared-fraction", "0.7", "--block-size", "4", "--max-num-seqs", "4",
                   "--max-num-batched-tokens", "16", "--concurrency", "6", "--env-json", str(tmp_path / "env.json")])
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and rec["requests"] == 12 and rec["concurrency"] == 6 and rec["generated_tokens"] == 60
    assert rec["decode_tokens_run"] >= 12 * 4 and rec["prompt_tokens_reused"] > 0 and rec["first_token_s_median"] > 0
    assert rec["pages"] == made["blocks"] == 4 * (-(-(30 + 5) // 4) + 1)
    assert (tmp_path / "env.json").exists()
    made["engine"].manager.check_invariants()
    assert len(made["engine"].stats.steps) > rec["steps"]  # the warm-up run came first and is not counted


def _fake_factory(made):
    def make(*args, num_blocks=None, block_size=16, config=None, **kw):
        eng, runner = fake_engine(num_pages=num_blocks or 64, page_size=block_size, max_num_seqs=config.max_num_seqs,
                                  budget=config.max_num_batched_tokens, watermark=kw.get("watermark", 0.01))
        runner.graph_steps = runner.mixed_graph_steps = 0
        runner.pools = types.SimpleNamespace(bytes_per_page=lambda *a: [64])
        made["engine"] = eng
        return eng

    return make


def test_generate_command_with_a_fake_engine(monkeypatch, capsys, tmp_path):
    made = {}
    monkeypatch.setattr(LLMEngine, "from_model_dir", staticmethod(_fake_factory(made)))
    (tmp_path / "prompts.txt").write_text("7 8 9\n\n4,5\n")
    rc = cli.main(["generate", "--model", "unused", "--prompt-ids", "1,2,3", "--prompt-file", str(tmp_path / "prompts.txt"), "--max-tokens", "5",
                   "--num-blocks", "32", "--block-size", "4", "--max-num-batched-tokens", "8", "--stop-token-ids", "", "--ignore-eos"])
    lines = [json.loads(line) for line in capsys.readouterr().out.strip().splitlines()]
    assert rc == 0 and [rec["prompt_ids"] for rec in lines] == [[1, 2, 3], [7, 8, 9], [4, 5]]
    assert [rec["output_ids"] for rec in lines] == [sequential(p, 5) for p in ([1, 2, 3], [7, 8, 9], [4, 5])]
    assert {rec["finish_reason"] for rec in lines} == {"length"}
    with pytest.raises(SystemExit):
        cli.main(["generate", "--model", "unused"])  # no prompt at all


def test_bench_command_refuses_a_batch_that_is_not_whole(monkeypatch, capsys):
    import torch

    made = {}
    monkeypatch.setattr(cli, "_model_for", lambda args: types.SimpleNamespace(
        spec=types.SimpleNamespace(vocab_size=50, run_order=()), parts=lambda: [], cache_needs=lambda: [], dtype=None))
    monkeypatch.setattr(LLMEngine, "for_model", staticmethod(_fake_factory(made)))
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a: None)
    monkeypatch.setattr(torch.cuda, "max_memory_allocated", lambda *a: 0)
    args = ["bench", "--random-config", "llama-3.2-1b", "--batch", "3", "--input-len", "10", "--block-size", "4", "--warmup", "2"]
    assert cli.main(args + ["--output-len", "30", "--steps", "5"]) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["batch"] == 3 and rec["steps"] == 5 and rec["tokens_per_s"] > 0
    assert made["engine"].manager._reserve == [0], "pages were held back in a pool sized for exactly this batch"
    with pytest.raises(SystemExit, match="output-len"):
        cli.main(args + ["--output-len", "6", "--steps", "20"])  # the requests end during the timed steps
    with pytest.raises(SystemExit, match="only 0 of 3"):
        cli.main(args + ["--output-len", "30", "--steps", "5", "--num-blocks", "2"])  # no request fits the pool at all
    with pytest.raises(SystemExit, match="preempted"):
        cli.main(args + ["--output-len", "30", "--steps", "25", "--num-blocks", "14"])  # all start, but they cannot all grow
