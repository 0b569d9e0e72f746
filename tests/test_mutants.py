"""Do the CPU tests notice faults?  Each mutant changes one line of the cache manager, the page pool, the
scheduler, the service order or the batch gathering in memory (the source is read, edited, compiled and put in
place of the method for the duration of one test), and at least one of the listed detectors has to fail.
The reference does the same to its block manager with four mutants (scripts/dev/mutation_check_block_manager.sh);
those four are the first four here.  No file is changed and no GPU is used."""

import inspect
import sys
import textwrap

import pytest

import tests.test_batch_host as batch_tests
import tests.test_cache_manager as cache_tests
import tests.test_cache_vs_golden as cache_golden
import tests.test_schedule_vs_golden as schedule_golden
import tests.test_scheduler as scheduler_tests
from dli_b200.cache.manager import CacheManager
from dli_b200.cache.page_pool import PagePool
from dli_b200.engine import batch as batch_mod
from dli_b200.engine.llm_engine import LLMEngine
from dli_b200.engine.ordering import ServiceOrder
from dli_b200.engine import scheduler as scheduler_mod
from dli_b200.engine.scheduler import Scheduler


def mutate(monkeypatch, owner, name, old, new):
    """Replace ``old`` by ``new`` in the source of ``owner.name`` and put the result in its place."""
    target = getattr(owner, name)
    src = textwrap.dedent(inspect.getsource(target))
    assert src.count(old) == 1, f"{name}: the line to change was not found exactly once"
    module = sys.modules[owner.__module__] if inspect.isclass(owner) else owner
    scope: dict = {}
    exec(compile(src.replace(old, new), f"<mutant of {name}>", "exec"), vars(module), scope)  # noqa: S102 - our own source, edited
    monkeypatch.setattr(owner, name, scope[name])
    for user in (batch_tests,):  # test modules that imported the function by name
        if getattr(user, name, None) is target:
            monkeypatch.setattr(user, name, scope[name])


# detectors: callables that raise when they notice something
def shadow_store():
    for seed in range(6):
        for caching, window in ((True, None), (False, None), (False, 7)):
            cache_tests.test_random_orders_keep_every_invariant(seed, caching, window)


def reference_traces():
    for case in cache_golden.CASES:
        cache_golden.test_same_answers_as_the_reference(case)


def fork_and_window():
    cache_tests.test_fork_shares_pages_and_the_first_append_copies_the_last_one()
    cache_tests.test_window_group_gives_pages_back_as_the_window_passes()
    cache_tests.test_watermark_holds_pages_back_for_running_requests()


class _Patch:  # the schedule test wants a monkeypatch fixture: give it one that undoes itself
    def __enter__(self):
        self.mp = pytest.MonkeyPatch()
        return self.mp

    def __exit__(self, *exc):
        self.mp.undo()


def reference_schedules():
    for case in schedule_golden.CASES:
        with _Patch() as mp:
            schedule_golden.test_same_steps_as_the_reference(case, False, mp)


def reference_schedules_ahead():
    for case in schedule_golden.CASES:
        with _Patch() as mp:
            schedule_golden.test_same_steps_as_the_reference(case, True, mp)


def scheduler_rules():
    scheduler_tests.test_pages_run_out_newest_is_preempted_and_recomputed()
    scheduler_tests.test_head_of_queue_is_not_overtaken()
    scheduler_tests.test_budget_and_request_cap_hold_every_step()
    scheduler_tests.test_a_preempted_request_comes_back_before_new_ones_of_its_class()
    scheduler_tests.test_interactive_goes_before_batch_and_aging_ends_the_wait()
    scheduler_tests.test_a_tenant_of_weight_two_gets_about_twice_the_tokens()
    scheduler_tests.test_an_idle_spell_earns_no_credit()


def gathered_arrays():
    for seed in range(6):
        batch_tests.test_gather_host_equals_a_per_token_restatement(seed)
    for seed in range(4):
        batch_tests.test_single_token_gather_equals_the_general_one(seed)


def engine_loop():
    scheduler_tests.test_one_step_ahead_in_steady_decode()
    scheduler_tests.test_an_arrival_stops_the_step_ahead()
    scheduler_tests.test_pages_written_by_steps_launched_ahead_are_found_again()
    for ahead in (False, True):
        scheduler_tests.test_stop_tokens_eos_and_length(ahead)
        scheduler_tests.test_batched_equals_sequential(ahead)
        for seed in range(8):
            scheduler_tests.test_random_scenarios(seed, ahead)


MUTANTS = {
    # the reference's four
    "no copy on write": (CacheManager, "append_slots", "and pool.ref[table[-1]] > 1]", "and pool.ref[table[-1]] > 1 and False]", [fork_and_window, reference_traces]),
    "pages shareable before they are computed": (CacheManager, "_index_full_pages", "full = req.num_computed // ps", "full = req.num_tokens // ps", [shadow_store, reference_traces]),
    "an idle page with children is evictable": (PagePool, "release", "if entry.children == 0:", "if entry.children >= 0:", [shadow_store, reference_traces]),
    "the prefix may cover the last token": (CacheManager, "_hits", "eligible = (len(token_ids) - 1) // self.page_size * self.page_size",
                                            "eligible = len(token_ids) // self.page_size * self.page_size", [reference_traces, shadow_store]),
    # more of the same kind
    "a freed page goes to the free list twice": (PagePool, "release", "        self.free.append(page)\n        return", "        self.free.append(page)\n        self.free.append(page)\n        return", [shadow_store]),
    "a hit is not revived before pages are taken": (CacheManager, "allocate", "pool.share(page)", "pass", [shadow_store, reference_traces]),
    "the watermark is ignored": (CacheManager, "_admissible", "(reserve if respect_watermark else 0)", "0", [fork_and_window, reference_traces]),
    "the window gives a page back one page early": (CacheManager, "mark_computed", "(num_computed - group.window + 1) // ps", "(num_computed - group.window + 1 + ps) // ps", [shadow_store, fork_and_window]),
    "eviction does not unlink the parent": (PagePool, "_evict", "parent.children -= 1", "pass", [reference_traces, shadow_store]),
    "a fork counts as a hit": (CacheManager, "fork", "found_by_hash=False", "found_by_hash=True", [reference_traces]),
    # scheduler and order
    "the oldest running request is the victim": (Scheduler, "_who_yields", "for c in reversed(self.running)", "for c in self.running", [reference_schedules, scheduler_rules]),
    "a step that preempted still admits": (Scheduler, "schedule", "if not step.out.preempted:", "if True:", [scheduler_rules, reference_schedules]),
    "the shortest waiting prompt is admitted first": (Scheduler, "_admit", "req = min(self.waiting, key=self.order.admission_key)",
                                                      "req = min(self.waiting, key=lambda r: len(r.prompt_ids))", [scheduler_rules, reference_schedules]),
    "the budget is not charged for the tokens given out": (scheduler_mod._Step, "give", "self.budget -= n", "self.budget -= 0", [scheduler_rules, reference_schedules]),
    "a request that lost its pages to an earlier one is served all the same": (Scheduler, "schedule", "if req.status is RequestStatus.RUNNING and", "if", [scheduler_rules, reference_schedules, engine_loop]),
    "new requests go before preempted ones": (ServiceOrder, "admission_key", "never_ran = 0 if req.num_preemptions else 1", "never_ran = 1 if req.num_preemptions else 0", [scheduler_rules, reference_schedules]),
    "aging never happens": (ServiceOrder, "service_class", "aged = self.steps - req.arrival_step >= self.aging_steps", "aged = False", [scheduler_rules, reference_schedules]),
    "weights are ignored": (ServiceOrder, "charge", "tokens / self.weights.get(tenant, 1.0)", "tokens", [scheduler_rules, reference_schedules]),
    "an idle tenant keeps its old clock": (ServiceOrder, "arrive", "max(self.clock(tenant), floor)", "self.clock(tenant)", [scheduler_rules, reference_schedules]),
    # the engine loop and the step launched ahead
    "a request that ends by length still gets a step ahead": (Scheduler, "schedule_ahead", "len(r.output_ids) + 1 < r.params.max_tokens", "len(r.output_ids) < r.params.max_tokens + 1", [engine_loop]),
    "the surplus token of a finished request is kept": (LLMEngine, "_resolve", "if req.is_finished:\n            continue", "if False:\n            continue", [engine_loop]),
    "a step is launched ahead although a request waits": (Scheduler, "schedule_ahead", "if self.waiting or not in_flight", "if not in_flight", [engine_loop, reference_schedules_ahead]),
    "slots taken for a step ahead that does not come about are forgotten": (LLMEngine, "_launch_ahead", "self._unknown.update(plan.unknown)", "pass", [engine_loop]),
    "an unknown token is never named": (LLMEngine, "_resolve", "self.manager.set_token(req.request_id, position, int(tok))", "pass", [engine_loop]),
    "the stop token is dropped from the output": (LLMEngine, "_append_token", "req.output_ids.append(tok)\n", "req.output_ids.append(tok)\n    if tok in req.params.stop_token_ids: req.output_ids.pop()\n", [engine_loop, reference_schedules]),
    # batch gathering
    "a slot at a page's edge is off by one": (batch_mod, "gather_host", "slots.append(pages * ps + positions % ps)",
                                              "slots.append(pages * ps + (positions + (positions % ps == ps - 1)) % ps)", [gathered_arrays]),
    "a decoded token's context is short by one": (batch_mod, "gather_single_tokens", "kv_len = starts + 1", "kv_len = starts", [gathered_arrays]),
    "wanted rows follow the batch's order, not the caller's": (batch_mod, "gather_host", "for i, e in enumerate(entries) for w in e.want]",
                                                               "for i, e in sorted(enumerate(entries), key=lambda p: place[p[0]]) for w in e.want]", [gathered_arrays]),
}


@pytest.mark.timeout(120)
@pytest.mark.parametrize("name", list(MUTANTS), ids=lambda n: n.replace(" ", "_"))
def test_mutant_is_noticed(name, monkeypatch):
    owner, method, old, new, detectors = MUTANTS[name]
    mutate(monkeypatch, owner, method, old, new)
    noticed = []
    for detect in detectors:
        try:
            detect()
        except Exception as exc:  # noqa: BLE001 - any failure counts as noticing
            noticed.append(f"{detect.__name__}: {type(exc).__name__}")
    assert noticed, f"'{name}' went through {[d.__name__ for d in detectors]} unnoticed"


def test_without_a_mutant_the_detectors_are_quiet():
    for detect in (shadow_store, reference_traces, fork_and_window, reference_schedules, reference_schedules_ahead, scheduler_rules, engine_loop, gathered_arrays):
        detect()
