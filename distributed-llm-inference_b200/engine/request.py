"""What the engine keeps per generation request.

The names are the reference's, because they are its Python API (src/dli/engine/request.py:13-66):
``Request`` with ``prompt_ids`` / ``output_ids`` / ``status`` / ``finish_reason``, the enums
``RequestStatus``, ``FinishReason`` and ``Priority``.  Sampler state is not an object here: a
request carries a ``seed``, and its n-th sampled token is drawn from (seed, n) on the device.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field

from ..sampling.params import SamplingParams


class Priority(enum.IntEnum):
    """Class of service.  The scheduler serves the smaller value first; BATCH work is promoted
    after it has waited long enough (``SchedulerConfig.aging_steps``)."""

    INTERACTIVE = 0
    BATCH = 1


class RequestStatus(enum.Enum):
    """WAITING: in the queue, also after a preemption, when everything is computed again.
    RUNNING: owns cache pages and takes part in every step.  FINISHED: gone from the scheduler."""

    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class FinishReason(str, enum.Enum):
    """Why a request ended.  STOP: it produced an end-of-sequence or stop id (kept in the output).
    LENGTH: ``max_tokens`` were generated.  ABORTED: the caller cancelled it.  CAPACITY: prompt plus
    ``max_tokens`` exceed the whole cache pool, so it was refused when it was added."""

    STOP = "stop"
    LENGTH = "length"
    ABORTED = "aborted"
    CAPACITY = "capacity"


@dataclass(eq=False)
class Request:
    # identity and input
    request_id: str
    prompt_ids: list[int]
    params: SamplingParams
    arrival: int  # order of add_request calls: ties between equals are broken by it
    seed: int = 0  # of this request's random stream
    priority: Priority = Priority.INTERACTIVE
    tenant: str = "default"  # whose share of the engine the tokens are charged to
    # progress
    output_ids: list[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: FinishReason | None = None
    num_computed_tokens: int = 0  # tokens whose keys and values are in the cache: the cache manager's own
    #                               count while the request holds pages, 0 again after a preemption
    num_preemptions: int = 0
    arrival_step: int = 0  # the scheduler's step count when the request was queued (its age starts there)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def is_finished(self) -> bool:
        return self.status is RequestStatus.FINISHED

    @property
    def all_token_ids(self) -> list[int]:
        """Prompt and generated ids as one new list (what a preempted request runs again)."""
        return self.prompt_ids + self.output_ids

    def token_slice(self, start: int, end: int) -> list[int]:
        """Ids at positions [start, end) of prompt + generated, without building the whole list."""
        split = len(self.prompt_ids)
        if start >= split:
            return self.output_ids[start - split : end - split]
        if end <= split:
            return self.prompt_ids[start:end]
        return self.prompt_ids[start:] + self.output_ids[: end - split]
