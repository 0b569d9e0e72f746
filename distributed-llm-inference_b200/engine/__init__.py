"""The engine above the model: everything that turns queued requests into steps.

    batch      host integers of a step -> one pinned upload -> StepBatch
    runner     ModelRunner.step: the step function; load_model / random_model
    graphs     captured pure-decode steps
    request    Request and its enums (the reference's API names)
    ordering   who is served first: classes, aging, tenants' shares
    scheduler  one batch per step under a token budget; preemption by recompute
    llm_engine LLMEngine: schedule, run, sample, retire; one decode step ahead
    generate   one request without the scheduler (greedy_generate, PagedSequence)
    workload   a closed set of requests with the times a load test asks for
"""

from .batch import StepBatch, StepEntry, build_batch
from .generate import PagedGeneration, PagedSequence, greedy_generate, paged_greedy_generate
from .llm_engine import LLMEngine, RequestOutput, StepStats
from .ordering import ServiceOrder
from .request import FinishReason, Priority, Request, RequestStatus
from .runner import ModelRunner, load_model, random_model, resolve_dtype
from .scheduler import ScheduledChunk, Scheduler, SchedulerConfig, SchedulerOutput
from .workload import ClosedLoopResult, percentile, run_closed_loop

__all__ = sorted(
    # the step function and what feeds it
    ["ModelRunner", "StepBatch", "StepEntry", "build_batch", "load_model", "random_model", "resolve_dtype"]
    # requests and their order
    + ["FinishReason", "Priority", "Request", "RequestStatus", "ServiceOrder"]
    # batching
    + ["ScheduledChunk", "Scheduler", "SchedulerConfig", "SchedulerOutput"]
    # the loop and its entry points
    + ["LLMEngine", "RequestOutput", "StepStats", "greedy_generate", "PagedGeneration", "PagedSequence", "paged_greedy_generate"]
    # measurement
    + ["ClosedLoopResult", "percentile", "run_closed_loop"]
)
