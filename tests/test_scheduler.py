"""The scheduler's decisions, with a model that has no tensors (no GPU)."""

import random

import pytest

from dli_b200 import SamplingParams
from dli_b200.engine import FinishReason, LLMEngine, Priority, SchedulerConfig
from tests.fake_runner import fake_engine, sequential


def prompts(rng, n, lo=1, hi=30):
    return [[rng.randrange(50) for _ in range(rng.randrange(lo, hi))] for _ in range(n)]


@pytest.mark.parametrize("ahead", [False, True])
def test_batched_equals_sequential(ahead):
    rng = random.Random(0)
    ps = prompts(rng, 12)
    eng, runner = fake_engine(ahead=ahead)
    assert eng.lookahead == ahead
    outs = eng.generate(ps, SamplingParams(max_tokens=20))
    assert outs == [sequential(p, 20) for p in ps]
    assert eng.manager.min_available_pages() == 64 and not eng.has_unfinished()
    eng.manager.check_invariants()


def test_budget_and_request_cap_hold_every_step():
    rng = random.Random(1)
    eng, runner = fake_engine(budget=16, max_num_seqs=3)
    eng.generate(prompts(rng, 9, 10, 40), SamplingParams(max_tokens=6))
    for step in runner.steps:
        assert sum(n for _, _, n, _ in step) <= 16 and len(step) <= 3
    assert any(n > 1 and not logits for step in runner.steps for _, _, n, logits in step), "no prompt was cut"


def test_long_prompt_is_cut_and_decodes_go_on_beside_it():
    eng, runner = fake_engine(budget=8)
    eng.add_request("short", [1, 2, 3], SamplingParams(max_tokens=12))
    eng.step()
    eng.add_request("long", list(range(40)), SamplingParams(max_tokens=2))
    for _ in range(5):
        eng.step()
    for step in runner.steps[1:6]:
        kinds = {rid: n for rid, _, n, _ in step}
        assert kinds["short"] == 1 and kinds["long"] == 7  # the running request first, the prompt takes the rest
    while eng.has_unfinished():
        eng.step()


def test_pages_run_out_newest_is_preempted_and_recomputed():
    rng = random.Random(2)
    ps = prompts(rng, 6, 8, 16)
    eng, runner = fake_engine(num_pages=14, page_size=4, budget=64, watermark=0.0)
    reqs = [eng.add_request(f"r{i}", p, SamplingParams(max_tokens=24)) for i, p in enumerate(ps)]
    seen_preempt_step_admits = False
    while eng.has_unfinished():
        before = {r.request_id for r in eng.scheduler.running}
        eng.step()
        st = eng.stats.steps[-1]
        if st.num_preempted:
            after = {r.request_id for r in eng.scheduler.running}
            assert after <= before, "a step that preempted also admitted"
            seen_preempt_step_admits = True
    assert seen_preempt_step_admits and sum(r.num_preemptions for r in reqs) > 0
    assert reqs[0].num_preemptions == 0, "the oldest request was preempted"
    assert [r.output_ids for r in reqs] == [sequential(p, 24) for p in ps]
    assert eng.manager.min_available_pages() == 14
    eng.manager.check_invariants()


def test_request_that_can_never_fit_is_refused():
    eng, _ = fake_engine(num_pages=4, page_size=4)
    r = eng.add_request("big", list(range(10)), SamplingParams(max_tokens=7))
    assert r.is_finished and r.finish_reason is FinishReason.CAPACITY and not eng.has_unfinished()
    ok = eng.add_request("fits", list(range(10)), SamplingParams(max_tokens=6))
    assert not ok.is_finished
    with pytest.raises(ValueError, match="duplicate"):
        eng.add_request("fits", [1])
    with pytest.raises(ValueError, match="non-empty"):
        eng.add_request("empty", [])


@pytest.mark.parametrize("ahead", [False, True])
def test_stop_tokens_eos_and_length(ahead):
    p = [3, 1, 4]
    full = sequential(p, 10)
    eng, _ = fake_engine(ahead=ahead)
    eng.eos = frozenset({full[4]})
    a = eng.add_request("a", p, SamplingParams(max_tokens=10))
    b = eng.add_request("b", p, SamplingParams(max_tokens=10, ignore_eos=True))
    c = eng.add_request("c", p, SamplingParams(max_tokens=10, ignore_eos=True, stop_token_ids=(full[2],)))
    while eng.has_unfinished():
        eng.step()
    first = full.index(full[4])
    assert a.output_ids == full[: first + 1] and a.finish_reason is FinishReason.STOP
    assert b.output_ids == full and b.finish_reason is FinishReason.LENGTH
    assert c.output_ids == full[: full.index(full[2]) + 1] and c.finish_reason is FinishReason.STOP


def test_abort_frees_everything_and_is_idempotent():
    eng, _ = fake_engine(budget=8)
    eng.add_request("a", list(range(30)), SamplingParams(max_tokens=5))
    eng.add_request("b", list(range(5)), SamplingParams(max_tokens=5))
    eng.step()
    assert eng.abort("a") and not eng.abort("a") and eng.abort("b") and not eng.abort("nobody")
    assert not eng.has_unfinished() and eng.manager.min_available_pages() == 64
    eng.manager.check_invariants()


def test_shared_prefix_starts_after_the_cached_pages():
    eng, runner = fake_engine(page_size=4, budget=64)
    stem = list(range(30))
    eng.generate([stem + [40]], SamplingParams(max_tokens=2))
    eng.generate([stem + [41, 42]], SamplingParams(max_tokens=2))
    first_chunk_of_second = runner.steps[2][0]
    assert first_chunk_of_second[1] == 28  # 7 full pages of the stem are reused
    assert eng.manager.stats.prompt_tokens_hit == 28


def test_head_of_queue_is_not_overtaken():
    eng, runner = fake_engine(num_pages=8, page_size=4, budget=64, watermark=0.0)
    eng.add_request("run", list(range(20)), SamplingParams(max_tokens=4))  # 6 pages at the end
    eng.step()
    eng.add_request("big", list(range(100, 116)), SamplingParams(max_tokens=4))  # does not fit beside it
    eng.add_request("small", [1], SamplingParams(max_tokens=1))  # would fit, but must wait its turn
    eng.step()
    assert {rid for rid, *_ in runner.steps[-1]} == {"run"}
    while eng.has_unfinished():
        eng.step()


@pytest.mark.parametrize("ahead", [False, True])
@pytest.mark.parametrize("seed", range(8))
def test_random_scenarios(seed, ahead):
    """Random pools, budgets, arrivals and aborts: outputs equal the sequential ones, every step
    keeps the invariants (checked inside the fake runner), nothing leaks.  With ``ahead`` the
    engine launches decode steps before it has read the ids of the step before."""
    rng = random.Random(seed)
    page = rng.choice([1, 2, 4, 8])
    pages = rng.randrange(12, 40)
    eng, runner = fake_engine(num_pages=pages, page_size=page, max_num_seqs=rng.randrange(1, 6),
                              budget=rng.randrange(1, 24), watermark=rng.choice([0.0, 0.1]),
                              prefix_caching=rng.random() < 0.7, ahead=ahead, eviction_policy=rng.choice(["lru", "cost"]),
                              tenant_weights={"t1": 2.0}, aging_steps=rng.choice([3, 200]))
    pending = []
    for i in range(14):
        stem = [7] * rng.randrange(0, 10)
        pending.append((f"r{i}", stem + [rng.randrange(50) for _ in range(rng.randrange(1, 12))], rng.randrange(1, 10)))
    live, aborted = {}, set()
    steps = 0
    while pending or eng.has_unfinished():
        if pending and rng.random() < 0.5:
            rid, p, mt = pending.pop()
            req = eng.add_request(rid, p, SamplingParams(max_tokens=mt), priority=rng.choice(list(Priority)),
                                  tenant=rng.choice(["t0", "t1", "t2"]))
            live[rid] = (req, p, mt)
        if live and rng.random() < 0.05:
            rid = rng.choice(sorted(live))
            if eng.abort(rid):
                aborted.add(rid)
        eng.step()
        steps += 1
        assert steps < 5000, "the engine does not make progress"
    for rid, (req, p, mt) in live.items():
        if rid in aborted:
            assert req.finish_reason is FinishReason.ABORTED
        elif req.finish_reason is FinishReason.CAPACITY:
            assert -(-(len(p) + mt) // page) > pages
        else:
            assert req.output_ids == sequential(p, mt)
    eng.manager.check_invariants()
    assert eng.manager.min_available_pages() == pages
    assert not eng._unknown


def test_one_step_ahead_in_steady_decode():
    """While everyone decodes and nobody waits, the next step is launched before the ids of the
    current one are read; a stop token costs one surplus token that is dropped; a request that
    ends by length is left out of the step ahead; an arrival makes the engine read first."""
    p, q = [3, 1, 4], [2, 7]
    eng, runner = fake_engine(ahead=True, page_size=2)
    stop_at = sequential(q, 6)[3]
    a = eng.add_request("a", p, SamplingParams(max_tokens=9))
    b = eng.add_request("b", q, SamplingParams(max_tokens=9, stop_token_ids=(stop_at,)))
    outs = eng.step()  # the prompts; the step after them is already launched
    assert len(runner.steps) == 2 and eng.steps_ahead == 1 and {o.request_id for o in outs} == {"a", "b"}
    assert all(n == 1 for _, _, n, _ in runner.steps[1])
    while not b.is_finished:
        eng.step()
    assert b.output_ids == sequential(q, 9, stop=(stop_at,)) and b.finish_reason is FinishReason.STOP
    surplus = [rid for rid, *_ in runner.steps[-1]]
    assert "b" in surplus, "the step ahead was launched before the stop token was read"
    late = eng.add_request("late", [9, 9, 9, 9, 9], SamplingParams(max_tokens=2))
    launched = len(runner.steps)
    eng.step()  # reads the step in flight; nothing new is launched ahead because a request waits
    assert len(runner.steps) == launched
    while eng.has_unfinished():
        eng.step()
    assert a.output_ids == sequential(p, 9) and late.output_ids == sequential([9] * 5, 2)
    # 'a' ends by length: its last token's step had no step ahead for it
    assert sum(1 for st in runner.steps for rid, *_ in st if rid == "a") == 9
    eng.manager.check_invariants()
    assert eng.manager.min_available_pages() == 64 and not eng._unknown


# ---- order among requests: classes, aging, tenants' shares


def tokens_by_tenant(runner, steps):
    served = {}
    for step in steps:
        for rid, _, n, _ in step:
            served[rid[0]] = served.get(rid[0], 0) + n
    return served


def test_tenants_with_queued_work_share_the_engine_whatever_the_order_of_arrival():
    eng, runner = fake_engine(max_num_seqs=2, budget=64)
    for i in range(12):  # all of A's requests arrive before any of B's
        eng.add_request(f"A{i}", [1, 2, i], SamplingParams(max_tokens=5), tenant="A")
    for i in range(12):
        eng.add_request(f"B{i}", [3, 4, i], SamplingParams(max_tokens=5), tenant="B")
    for _ in range(40):
        eng.step()
    served = tokens_by_tenant(runner, runner.steps)
    assert abs(served["A"] - served["B"]) <= 8, served  # one request's worth at most
    while eng.has_unfinished():
        eng.step()


def test_a_tenant_of_weight_two_gets_about_twice_the_tokens():
    eng, runner = fake_engine(max_num_seqs=3, budget=64, tenant_weights={"A": 2.0, "B": 1.0})
    for i in range(30):
        eng.add_request(f"A{i}", [1, i], SamplingParams(max_tokens=8), tenant="A")
        eng.add_request(f"B{i}", [2, i], SamplingParams(max_tokens=8), tenant="B")
    for _ in range(60):
        eng.step()
    served = tokens_by_tenant(runner, runner.steps)
    assert 1.5 < served["A"] / served["B"] < 2.6, served
    assert eng.scheduler.tenant_clock("A") == pytest.approx(served["A"] / 2.0)
    while eng.has_unfinished():
        eng.step()


def test_an_idle_spell_earns_no_credit():
    eng, runner = fake_engine(max_num_seqs=2, budget=64)
    for i in range(10):
        eng.add_request(f"A{i}", [1, i], SamplingParams(max_tokens=4), tenant="A")
    for _ in range(12):
        eng.step()  # B has been idle all this time
    for i in range(10):
        eng.add_request(f"B{i}", [2, i], SamplingParams(max_tokens=4), tenant="B")
        eng.add_request(f"A{10 + i}", [1, 10 + i], SamplingParams(max_tokens=4), tenant="A")
    assert eng.scheduler.tenant_clock("B") == eng.scheduler.tenant_clock("A") > 0
    mark = len(runner.steps)
    for _ in range(20):
        eng.step()
    served = tokens_by_tenant(runner, runner.steps[mark:])
    assert abs(served["A"] - served["B"]) <= 12, served  # B does not take the engine over to catch up
    while eng.has_unfinished():
        eng.step()


def test_interactive_goes_before_batch_and_aging_ends_the_wait():
    eng, runner = fake_engine(max_num_seqs=1, budget=64, aging_steps=6)
    eng.add_request("old_batch", [5, 5], SamplingParams(max_tokens=2), priority=Priority.BATCH)
    order = []
    for i in range(12):  # an interactive request arrives before every step
        eng.add_request(f"i{i}", [i, 1], SamplingParams(max_tokens=1))
        eng.step()
        order += [rid for rid, *_ in runner.steps[-1] if rid not in order]
    assert order[0] == "i0", "a batch request was admitted in front of an interactive one"
    assert "old_batch" in order, "the batch request starved"
    assert 5 <= order.index("old_batch") <= 7  # after aging_steps steps it counts as interactive, and it is the oldest
    while eng.has_unfinished():
        eng.step()


def test_running_interactive_requests_get_the_budget_before_running_batch_ones():
    eng, runner = fake_engine(max_num_seqs=4, budget=2)
    eng.add_request("b0", [1], SamplingParams(max_tokens=30), priority=Priority.BATCH)
    eng.add_request("b1", [2], SamplingParams(max_tokens=30), priority=Priority.BATCH)
    eng.step()
    eng.add_request("i0", [3], SamplingParams(max_tokens=6))
    eng.step()  # no room in the budget: the two batch requests take it, i0 waits
    eng.step()
    for step in runner.steps[3:6]:
        assert step[0][0] == "i0", step  # once it runs, it is served first, and one batch request sits out
        assert len(step) == 2
    while eng.has_unfinished():
        eng.step()


def test_a_preempted_request_comes_back_before_new_ones_of_its_class():
    eng, runner = fake_engine(num_pages=6, page_size=4, max_num_seqs=4, budget=64, watermark=0.0, prefix_caching=False)
    a = eng.add_request("a", list(range(8)), SamplingParams(max_tokens=14))
    b = eng.add_request("b", list(range(20, 28)), SamplingParams(max_tokens=14))
    while not b.num_preemptions:
        eng.step()
    eng.add_request("new", [9], SamplingParams(max_tokens=1))
    assert eng.scheduler.order.admission_key(b) < eng.scheduler.order.admission_key(eng.scheduler._known["new"])
    while eng.has_unfinished():
        eng.step()
    assert a.output_ids == sequential(list(range(8)), 14) and b.output_ids == sequential(list(range(20, 28)), 14)


def test_scheduler_config_checks_its_values():
    with pytest.raises(ValueError, match="aging_steps"):
        SchedulerConfig(aging_steps=0)
    with pytest.raises(ValueError, match="positive"):
        SchedulerConfig(tenant_weights={"A": 0.0})
    with pytest.raises(ValueError, match=">= 1"):
        SchedulerConfig(max_num_seqs=0)


def test_a_request_that_needs_the_watermark_pages_runs_when_it_is_alone():
    """10 pages, 2 of them held back for running requests: a request of 9 pages passes the
    capacity check, can never be admitted beside the watermark, and must still run."""
    eng, runner = fake_engine(num_pages=10, page_size=4, budget=64, watermark=0.2)
    small = eng.add_request("small", [1, 2, 3], SamplingParams(max_tokens=4))
    big = eng.add_request("big", list(range(30)), SamplingParams(max_tokens=6))  # 36 tokens = 9 pages
    steps = 0
    while eng.has_unfinished():
        eng.step()
        steps += 1
        assert steps < 100, "the big request waits for ever"
    assert big.output_ids == sequential(list(range(30)), 6) and small.output_ids == sequential([1, 2, 3], 4)
    first_big = next(i for i, st in enumerate(runner.steps) if any(rid == "big" for rid, *_ in st))
    assert all(rid != "small" for rid, *_ in runner.steps[first_big]), "it was admitted beside a running request"
    eng.manager.check_invariants()


# ---- one request stepped by hand on a shared runner


def test_paged_sequence_and_paged_greedy_generate_reuse_the_prefix():
    import numpy as np

    from dli_b200.engine import PagedSequence, paged_greedy_generate
    from tests.fake_runner import FakeRunner

    runner = FakeRunner(num_pages=40, page_size=4, watermark=0.0)
    pick = lambda row: int(np.argmax(row))  # noqa: E731
    stem = list(range(10, 23))  # 13 tokens: three full pages
    p1, p2 = stem + [1, 2], stem + [3]
    runner.prompts.update(a=p1, b=p2)
    first = paged_greedy_generate(runner, "a", p1, 7, pick=pick)
    assert first.tokens == sequential(p1, 7) and first.num_cached_prompt_tokens == 0 and not runner.manager.has_request("a")
    second = paged_greedy_generate(runner, "b", p2, 5, pick=pick, release=False)
    assert second.tokens == sequential(p2, 5) and second.num_cached_prompt_tokens == 12
    assert ("b", 12, 2) in runner.stepped, "the prompt's rest did not start behind the reused pages"
    # an end-of-sequence id ends the generation and is kept
    stop = sequential(p1, 7)[2]
    runner.prompts["c"] = p1
    assert paged_greedy_generate(runner, "c", p1, 7, eos_token_ids={stop}, pick=pick).tokens == sequential(p1, 7)[:3]
    # feeding forced tokens by hand: the logits after each are those of the history so far
    seq = PagedSequence(runner, "b")
    hist = p2 + second.tokens[:-1]  # the last sampled token was never fed
    for forced in (7, 7, 9):
        row = seq.feed(forced)
        hist.append(forced)
        assert pick(row) == sequential(hist, 1)[0]
    with pytest.raises(KeyError):
        PagedSequence(runner, "nobody")
    runner.manager.free("b")
    runner.manager.check_invariants()
    assert runner.manager.min_available_pages() == 40


def test_a_stalled_engine_ends_the_loop_instead_of_stepping_for_ever():
    from dli_b200.engine import run_closed_loop

    for drive in (lambda e: e.generate([[1, 2, 3]], SamplingParams(max_tokens=2)),
                  lambda e: run_closed_loop(e, [[1, 2, 3]], SamplingParams(max_tokens=2))):
        eng, _ = fake_engine()
        eng.manager.can_allocate = lambda *a, **k: False  # a fault in the rules of admission, made up for the test
        with pytest.raises(RuntimeError, match="no progress"):
            drive(eng)
    eng, _ = fake_engine()
    assert not eng.is_stalled()
    eng.generate([[1, 2, 3]], SamplingParams(max_tokens=2))
    assert not eng.is_stalled()


def test_an_arrival_stops_the_step_ahead():
    eng, runner = fake_engine(ahead=True)
    eng.add_request("a", [1, 2, 3], SamplingParams(max_tokens=20))
    eng.step(), eng.step()  # steady decoding: every step is launched before the ids of the one before are read
    assert eng.steps_ahead == 2
    launched = len(runner.steps)
    eng.add_request("late", [4, 5], SamplingParams(max_tokens=3))
    eng.step()  # reads the step in flight; nothing is launched ahead, because a request waits
    assert len(runner.steps) == launched
    eng.step()  # the scheduler decides again: the newcomer's prompt beside the decoded token
    assert {rid for rid, *_ in runner.steps[-1]} == {"a", "late"}
    while eng.has_unfinished():
        eng.step()


def test_pages_written_by_steps_launched_ahead_are_found_again():
    """Tokens that ran before the host knew their ids are named afterwards (set_token), so their pages
    enter the prefix index like any others."""
    eng, _ = fake_engine(ahead=True, page_size=4, budget=64)
    prompt = [1, 2, 3]
    out = eng.generate([prompt], SamplingParams(max_tokens=14))[0]  # 16 tokens computed: four full pages
    assert eng.steps_ahead > 5
    before = eng.manager.stats.prompt_tokens_hit
    eng.generate([prompt + out], SamplingParams(max_tokens=1))
    assert eng.manager.stats.prompt_tokens_hit - before == 16


@pytest.mark.parametrize("ahead", [False, True])
def test_a_device_wait_that_ran_out_fails_the_steps_requests_and_leaves_the_engine_usable(ahead):
    """The runner reports that a kernel gave up a bounded wait: the step's tokens are not handed out, its
    requests are aborted, no page they wrote stays in the prefix index, the error reaches the caller,
    and requests that come afterwards run as if nothing had happened."""
    eng, runner = fake_engine(num_pages=64, page_size=4, ahead=ahead)
    failing = {"now": False}

    def check_device_errors():
        if failing["now"]:
            failing["now"] = False
            raise RuntimeError("a device-side wait ran out")

    runner.check_device_errors = check_device_errors
    prompts = [[1, 2, 3, 4, 5, 6, 7, 8, 9], [11, 12, 13]]
    reqs = [eng.add_request(f"r{i}", p, SamplingParams(max_tokens=12)) for i, p in enumerate(prompts)]
    for _ in range(3):
        eng.step()
    before = [list(r.output_ids) for r in reqs]
    failing["now"] = True
    with pytest.raises(RuntimeError, match="wait ran out"):
        eng.step()
    assert [r.output_ids for r in reqs] == before, "tokens of the failed step were handed out"
    assert all(r.finish_reason is FinishReason.ABORTED for r in reqs) and not eng.has_unfinished()
    runner.manager.check_invariants()
    group = runner.manager.stats().groups[0]
    assert group.used_pages == 0 and group.cached_idle_pages == 0, "pages of the failed step stayed indexed"
    # the engine goes on: the same prompt again is computed from its first token (no prefix hit) and is right
    steps_before = len(runner.steps)
    assert eng.generate([prompts[0]], SamplingParams(max_tokens=6)) == [sequential(prompts[0], 6)]
    assert runner.steps[steps_before][0][1:3] == (0, len(prompts[0])), "the prompt was served from pages of the failed step"


def test_a_sampler_with_state_slots_is_told_each_requests_seed_and_draws_and_counts_on_by_itself():
    """The engine's side of sampling by state slot: every admitted request is bound to its slot with its parameters, its
    seed and the draws it has made (none at first; after a preemption as many as it has tokens), every step passes the
    slots of its rows, and the sampler counts the draws itself.  The fake below keeps the table on the host and records,
    per request seed, which draw produced which token: every request must have used draws 0, 1, 2, ... exactly once each,
    in a pool so small that requests are preempted, with steps launched ahead."""
    from tests.fake_runner import AheadRunner, FakeTokens

    class SlotSampler:
        def __init__(self):
            self.state = {}  # slot -> [seed, draws, greedy]
            self.used = {}  # seed -> draw indices, in the order they were made

        def bind(self, slot, params, seed, draws):
            self.state[slot] = [seed, draws, params.greedy]

        def sample_slots_async(self, logits, slots, all_greedy):
            assert len(slots) == len(logits)
            for slot in slots:
                seed, draws, greedy = self.state[slot]
                if not greedy:
                    assert not all_greedy
                    self.used.setdefault(seed, []).append(draws)
                    self.state[slot][1] = draws + 1
            return FakeTokens(logits)

        sample_async = None  # (present, so the engine may launch a step ahead)

    runner = AheadRunner(10, 4, max_requests=4, prefix_caching=True, watermark=0.0)
    sampler = SlotSampler()
    eng = LLMEngine(runner, SchedulerConfig(4, 16), sampler=sampler)
    assert eng.lookahead
    rng = random.Random(5)
    reqs = []
    for i in range(6):
        greedy = i == 2
        reqs.append(eng.add_request(f"r{i}", [rng.randrange(50) for _ in range(rng.randrange(3, 11))],
                                    SamplingParams(max_tokens=rng.randrange(4, 9), temperature=0.0 if greedy else 0.8, seed=1000 + i)))
    while eng.has_unfinished():
        eng.step()
        assert not eng.is_stalled()
    assert sum(s.num_preempted for s in eng.stats.steps) > 0 and eng.steps_ahead > 0
    for i, r in enumerate(reqs):
        assert r.output_ids == sequential(r.prompt_ids, r.params.max_tokens)
        if i == 2:
            assert 1002 not in sampler.used
        else:  # a step launched ahead may have drawn once more than the request kept
            draws = sampler.used[1000 + i]
            assert draws[: len(r.output_ids)] == list(range(len(r.output_ids))) and len(draws) <= len(r.output_ids) + 1, (i, draws)
