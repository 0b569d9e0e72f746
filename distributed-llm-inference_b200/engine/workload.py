"""Runs a closed set of requests through an engine and keeps the times a load test asks for.

Closed loop, as the reference's load generator defines it (benchmarks/methodology.md:69-77):
``concurrency`` requests are in flight; when one finishes, the next prompt is submitted.  Time to
the first token is counted from a request's own submission, time per output token from its first
token to its last.  With ``concurrency=None`` every request is queued at the start.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Sequence

from ..sampling import SamplingParams
from .request import Request


@dataclass
class ClosedLoopResult:
    seconds: float
    requests: list[Request]
    submitted_s: dict[str, float] = field(default_factory=dict)
    first_token_s: dict[str, float] = field(default_factory=dict)  # since the start of the run
    done_s: dict[str, float] = field(default_factory=dict)
    steps: int = 0

    def time_to_first_token(self) -> list[float]:
        """Per request that produced a token: first token minus its own submission, sorted."""
        return sorted(self.first_token_s[r] - self.submitted_s[r] for r in self.first_token_s)

    def time_per_output_token(self) -> list[float]:
        """Per request with at least two tokens: (last token - first token) / (tokens - 1), sorted."""
        out = []
        for req in self.requests:
            rid, n = req.request_id, len(req.output_ids)
            if n > 1 and rid in self.done_s and rid in self.first_token_s:
                out.append((self.done_s[rid] - self.first_token_s[rid]) / (n - 1))
        return sorted(out)


def percentile(sorted_values: Sequence[float], q: float) -> float | None:
    """The value at fraction ``q`` of a sorted list (nearest rank); None for an empty one."""
    if not sorted_values:
        return None
    return sorted_values[min(len(sorted_values) - 1, max(0, int(round(q * (len(sorted_values) - 1)))))]


def run_closed_loop(engine, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams], *,
                    concurrency: int | None = None, name: str = "w", clock: Callable[[], float] = time.perf_counter,
                    synchronize: Callable[[], None] | None = None) -> ClosedLoopResult:
    """Submit ``prompts`` to ``engine`` (an LLMEngine), at most ``concurrency`` at a time, and step
    it until all are finished.  ``synchronize`` (the device's, if any) brackets the timed region."""
    if concurrency is not None and concurrency < 1:
        raise ValueError("concurrency must be at least 1")
    per = list(params) if isinstance(params, Sequence) else [params] * len(prompts)
    if len(per) != len(prompts):
        raise ValueError("one SamplingParams per prompt, or one for all")
    limit = len(prompts) if concurrency is None else concurrency
    waiting = deque(range(len(prompts)))
    reqs: list[Request | None] = [None] * len(prompts)
    res = ClosedLoopResult(0.0, [])
    live: set[str] = set()

    if synchronize:
        synchronize()
    t0 = clock()

    def submit_some() -> None:
        while waiting and len(live) < limit:
            i = waiting.popleft()
            rid = f"{name}-{i}"
            res.submitted_s[rid] = clock() - t0
            req = reqs[i] = engine.add_request(rid, prompts[i], per[i])
            if req.is_finished:  # refused at once: it could never fit
                res.done_s[rid] = res.submitted_s[rid]
            else:
                live.add(rid)

    submit_some()
    while engine.has_unfinished():
        outputs = engine.step()
        res.steps += 1
        now = clock() - t0
        for out in outputs:
            if out.new_token_ids:
                res.first_token_s.setdefault(out.request_id, now)
            if out.finished:
                res.done_s[out.request_id] = now
                live.discard(out.request_id)
        for rid in [r for r in live if reqs[int(r.rsplit("-", 1)[1])].is_finished]:  # ended without an output (aborted elsewhere)
            res.done_s.setdefault(rid, now)
            live.discard(rid)
        submit_some()
        if getattr(engine, "is_stalled", lambda: False)():
            raise RuntimeError("the engine makes no progress: requests wait, nothing runs and nothing could be scheduled")
    if synchronize:
        synchronize()
    res.seconds = clock() - t0
    res.requests = [r for r in reqs if r is not None]
    return res
