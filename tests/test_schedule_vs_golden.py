"""The scheduler and the engine loop against the reference's own: the events of
tests/golden/schedule_trace.json (made by tests/golden/make_schedule_trace.py from ``dli.engine.LLMEngine``
with the reference's fake model) are run here and every step is compared: the batch that was chosen
(request, start, tokens, whether a token is sampled), how many were preempted, the tokens and finish
reasons that came out.  With the step launched ahead, the tokens of every step are compared.  No GPU."""

import hashlib
import json
from pathlib import Path

import pytest

from dli_b200 import Priority, SamplingParams
from dli_b200.engine import LLMEngine, SchedulerConfig
from tests import fake_runner

CASES = json.loads((Path(__file__).resolve().parent / "golden" / "schedule_trace.json").read_text())


def reference_next_token(history) -> int:
    """The rule of the reference's fake model (tests/unit/engine/fake.py:21-23), so that stop ids and
    the contents of indexed pages are the same as in the recorded run."""
    digest = hashlib.blake2b(bytes(str(list(history)), "ascii"), digest_size=8).digest()
    return int.from_bytes(digest, "little") % 50


@pytest.mark.parametrize("ahead", [False, True], ids=["read_first", "one_step_ahead"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"seed{c['seed']}-{c['num_blocks']}x{c['block_size']}")
def test_same_steps_as_the_reference(case, ahead, monkeypatch):
    monkeypatch.setattr(fake_runner, "next_token", reference_next_token)
    runner = (fake_runner.AheadRunner if ahead else fake_runner.FakeRunner)(
        case["num_blocks"], case["block_size"], max_requests=case["max_num_seqs"], prefix_caching=case["prefix_caching"],
        watermark=case["watermark"], eviction_policy=case["policy"])
    config = SchedulerConfig(case["max_num_seqs"], case["budget"], tenant_weights=case["tenant_weights"], aging_steps=case["aging_steps"])
    eng = LLMEngine(runner, config, sampler=fake_runner.AheadSampler() if ahead else fake_runner.FakeSampler())
    assert eng.lookahead == ahead
    reqs, cancelled, expected = {}, set(), {}
    for i, step in enumerate(case["steps"]):
        for r in step["add"]:
            reqs[r["id"]] = eng.add_request(r["id"], r["prompt"], SamplingParams(max_tokens=r["max_tokens"], stop_token_ids=tuple(r["stop"])),
                                            priority=Priority(r["priority"]), tenant=r["tenant"])
        for rid in step["abort"]:
            assert eng.abort(rid), f"step {i}: {rid} was still alive in the reference"
            cancelled.add(rid)
        for rid, tok, reason in step["out"]:
            expected.setdefault(rid, [[], None])[0].append(tok)
            expected[rid][1] = reason
        launched = len(runner.steps)
        outs = eng.step()
        if ahead:
            continue  # a request that arrives while a step launched ahead is in flight starts one step later: compared at the end
        got = [[o.request_id, o.new_token_ids[0], o.finish_reason.value if o.finish_reason else None] for o in outs]
        chunks = [[rid, start, n, int(logits)] for rid, start, n, logits in runner.steps[-1]] if len(runner.steps) > launched else []
        assert chunks == step["chunks"], f"step {i}: another batch than the reference's"
        assert eng.stats.steps[-1].num_preempted == step["preempted"], f"step {i}"
        assert got == step["out"], f"step {i}"
    while eng.has_unfinished():
        eng.step()
    for rid, req in reqs.items():
        want_tokens, want_reason = expected.get(rid, [[], None])
        if rid in cancelled:  # cancelled at the same moment, possibly a token earlier in its life
            assert req.finish_reason.value == "aborted" and req.output_ids == want_tokens[: len(req.output_ids)], rid
        else:
            assert (req.output_ids, req.finish_reason.value) == (want_tokens, want_reason), rid
    runner.manager.check_invariants()
    assert runner.manager.min_available_pages() == case["num_blocks"]
