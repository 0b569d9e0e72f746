"""A generation request and its progress (src/dli/engine/request.py:13-66)."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, IntEnum

from ..sampling.params import SamplingParams


class RequestStatus(Enum):
    WAITING = "waiting"  # queued, or preempted and waiting to be recomputed
    RUNNING = "running"  # holds cache pages and is scheduled every step
    FINISHED = "finished"


class FinishReason(str, Enum):
    STOP = "stop"  # emitted an end-of-sequence or stop token
    LENGTH = "length"  # reached max_tokens
    ABORTED = "aborted"
    CAPACITY = "capacity"  # can never fit in the cache pool; never ran


class Priority(IntEnum):
    """Scheduling class of a request; the lower value is served first (src/dli/engine/request.py:27-31)."""

    INTERACTIVE = 0
    BATCH = 1


@dataclass(eq=False)
class Request:
    """``num_computed_tokens`` counts tokens whose keys and values are in the cache; it equals
    the cache manager's count while the request holds pages and drops to 0 at preemption."""

    request_id: str
    prompt_ids: list[int]
    params: SamplingParams
    arrival: int
    seed: int = 0
    priority: Priority = Priority.INTERACTIVE
    tenant: str = "default"  # whose share of the engine the request's tokens are charged to
    arrival_step: int = 0  # the scheduler's step count when the request was queued (for aging)
    output_ids: list[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: FinishReason | None = None
    num_computed_tokens: int = 0
    num_preemptions: int = 0

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_ids + self.output_ids

    def token_slice(self, start: int, end: int) -> list[int]:
        """Tokens at positions [start, end) of prompt + generated, without building the whole list."""
        n = len(self.prompt_ids)
        if start >= n:
            return self.output_ids[start - n : end - n]
        if end <= n:
            return self.prompt_ids[start:end]
        return self.prompt_ids[start:] + self.output_ids[: end - n]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def is_finished(self) -> bool:
        return self.status is RequestStatus.FINISHED
