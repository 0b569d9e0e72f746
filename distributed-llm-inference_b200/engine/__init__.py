from .batch import StepBatch, StepEntry, build_batch
from .generate import PagedGeneration, PagedSequence, greedy_generate, paged_greedy_generate
from .llm_engine import LLMEngine, RequestOutput, StepStats
from .request import FinishReason, Priority, Request, RequestStatus
from .runner import ModelRunner, load_model, random_model, resolve_dtype
from .scheduler import ScheduledChunk, Scheduler, SchedulerConfig, SchedulerOutput
from .workload import ClosedLoopResult, percentile, run_closed_loop

__all__ = [
    "ClosedLoopResult", "FinishReason", "LLMEngine", "ModelRunner", "PagedGeneration", "PagedSequence", "Priority", "Request", "RequestOutput", "RequestStatus", "ScheduledChunk",
    "Scheduler", "SchedulerConfig", "SchedulerOutput", "StepBatch", "StepEntry", "StepStats", "build_batch",
    "greedy_generate", "load_model", "paged_greedy_generate", "random_model", "resolve_dtype", "run_closed_loop",
]
