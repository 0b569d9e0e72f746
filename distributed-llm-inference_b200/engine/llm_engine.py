"""LLMEngine: schedule, run one batched step, sample, update requests, retire the finished.

Names and meanings follow src/dli/engine/engine.py:62-246 (for_model, add_request,
step, generate, abort, has_unfinished, StepStats).  Token ids in, token ids out.

One step ahead.  While every running request is decoding and nobody waits, the engine
launches the next step before it reads the ids the current one sampled: the ids stay on the
device, the next step takes them from there, and the host reads them one step late, while
the device is already busy.  ``step()`` still returns the tokens of exactly one model step.
A request that turns out to have ended (a stop token) has one surplus token computed, which
is dropped; a request that ends by length is left out of the step ahead.  Whenever a request
waits, a prompt is in portions, or a page is missing, the engine reads first and schedules
then, as the reference does at every step.
"""

from __future__ import annotations

import itertools
import random
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Collection, Iterable, Protocol, Sequence

from ..sampling import SamplingParams
from .request import FinishReason, Priority, Request
from .scheduler import ScheduledChunk, Scheduler, SchedulerConfig


@dataclass(frozen=True)
class RequestOutput:
    request_id: str
    new_token_ids: list[int]
    finished: bool
    finish_reason: FinishReason | None


@dataclass(frozen=True)
class StepStats:
    """Shape and timing (seconds) of one step (src/dli/engine/engine.py:39-54)."""

    num_seqs: int
    num_batched_tokens: int
    num_prefill_tokens: int
    num_decode_tokens: int
    num_preempted: int
    schedule_s: float
    forward_s: float
    postprocess_s: float

    @property
    def total_s(self) -> float:
        return self.schedule_s + self.forward_s + self.postprocess_s


@dataclass
class _Counters:
    steps: list[StepStats] = field(default_factory=list)


class Runner(Protocol):
    """What the engine needs of the thing that runs a step (src/dli/engine/runner.py:18-25)."""

    manager: object

    def start_request(self, request_id: str, slot: int) -> None: ...

    def execute(self, chunks: Sequence[ScheduledChunk]):
        """Run the chunks as one batch; afterwards their tokens count as computed in the cache
        manager.  Returns one logits row per chunk with ``needs_logits``, in the chunks' order."""


class _Ready:
    """Token ids that are already on the host (a sampler without ``sample_async``)."""

    device_ids = None

    def __init__(self, ids) -> None:
        self._ids = list(ids)

    def result(self) -> list[int]:
        return self._ids


@dataclass
class _InFlight:
    """A step that was launched and whose sampled ids have not been read."""

    chunks: list[ScheduledChunk]
    sampling: list[Request]  # who gets a token, in the order of the sampled rows
    tokens: object  # PendingTokens or _Ready
    num_preempted: int
    launch_s: float


class LLMEngine:
    def __init__(self, runner: Runner, config: SchedulerConfig | None = None, *, sampler=None,
                 eos_token_ids: Collection[int] = (), seed: int = 0, lookahead: bool = True) -> None:
        self.runner = runner
        self.manager = runner.manager
        self.scheduler = Scheduler(config or SchedulerConfig(), self.manager)
        self.sampler = sampler
        self.eos = frozenset(eos_token_ids)
        self._rng = random.Random(seed)
        self._arrivals = itertools.count()
        self.stats = _Counters()
        # one step ahead needs a runner that takes token ids from the device and a sampler that leaves them there
        self.lookahead = bool(lookahead and getattr(runner, "takes_token_source", False) and hasattr(sampler, "sample_async"))
        self.steps_ahead = 0  # steps that were launched before the ids they run on were read
        # a sampler with a table of state slots keeps each request's parameters, seed and draw count on the device
        self._by_slot = getattr(sampler, "state", None) is not None and hasattr(sampler, "sample_slots_async")
        self._inflight: _InFlight | None = None
        self._unknown: dict[str, int] = {}  # request -> position whose id the cache manager does not know yet
        self._preempted_for_nothing = 0  # requests preempted by a scheduling round that produced no batch

    # ------------------------------------------------------------ construction

    @classmethod
    def for_model(cls, model, *, num_blocks: int | None = None, kv_cache_gb: float | None = None, block_size: int = 16,
                  config: SchedulerConfig | None = None, enable_prefix_caching: bool = True, watermark: float = 0.01,
                  eos_token_ids: Collection[int] = (), seed: int = 0, lookahead: bool = True,
                  eviction_policy: str = "lru") -> "LLMEngine":
        """An engine around a loaded model.  The cache pool has ``num_blocks`` pages of
        ``block_size`` tokens, or as many as ``kv_cache_gb`` GiB hold (default 1 GiB).
        ``eviction_policy``: which idle prefix page goes first, "lru" or "cost"
        (src/dli/engine/engine.py:92-107, src/dli/kv/eviction.py:167)."""
        from ..sampling import Sampler
        from .runner import ModelRunner

        config = config or SchedulerConfig()
        if num_blocks is not None and kv_cache_gb is not None:
            raise ValueError("give num_blocks or kv_cache_gb, not both")
        if num_blocks is None:
            num_blocks = ModelRunner.pages_for_budget(model, (kv_cache_gb or 1.0) * 2**30, block_size)
        runner = ModelRunner(model, num_pages=num_blocks, page_size=block_size, max_requests=config.max_num_seqs,
                             enable_prefix_caching=enable_prefix_caching, watermark=watermark, eviction_policy=eviction_policy)
        sampler = Sampler(model.device, max_requests=config.max_num_seqs)  # a slot of sampler state beside each request's cache state
        return cls(runner, config, sampler=sampler, eos_token_ids=eos_token_ids, seed=seed, lookahead=lookahead)

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, *, dtype: str = "auto", device: str = "cuda:0", **kwargs) -> "LLMEngine":
        from .runner import load_model

        return cls.for_model(load_model(model_dir, dtype, device), **kwargs)

    # ------------------------------------------------------------ API

    def add_request(self, request_id: str, prompt_ids: Sequence[int], params: SamplingParams | None = None, *,
                    priority: Priority = Priority.INTERACTIVE, tenant: str = "default") -> Request:
        """Queue a request.  One that can never fit finishes at once with reason ``capacity``.
        ``priority`` and ``tenant`` decide its place among the others (see the scheduler)."""
        if not prompt_ids:
            raise ValueError("prompt must be non-empty")
        params = params or SamplingParams()
        seed = params.seed if params.seed is not None else self._rng.getrandbits(63)
        req = Request(request_id, [int(t) for t in prompt_ids], params, next(self._arrivals), seed=seed,
                      priority=Priority(priority), tenant=tenant)
        self.scheduler.add(req)
        return req

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id) is not None

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished

    def step(self) -> list[RequestOutput]:
        """Advance by one model step; the tokens it produced, one RequestOutput per request."""
        t0 = time.perf_counter()
        flight, self._inflight = self._inflight, None
        self._preempted_for_nothing = 0
        if flight is None:
            flight = self._launch_scheduled()
        t1 = time.perf_counter()
        if flight is None:
            self.stats.steps.append(StepStats(0, 0, 0, 0, self._preempted_for_nothing, t1 - t0, 0.0, 0.0))
            return []
        ahead = self._launch_ahead(flight) if self.lookahead else None
        t2 = time.perf_counter()
        tokens = flight.tokens.result()
        self._check_device(flight, ahead)
        t3 = time.perf_counter()
        outputs = self._resolve(flight, tokens)
        if ahead is not None and self.scheduler.running:
            self._inflight = ahead  # (if nobody is left, its surplus tokens are simply never read)
        t4 = time.perf_counter()
        batched = sum(c.num_tokens for c in flight.chunks)
        prefill = sum(c.num_tokens for c in flight.chunks if c.num_tokens > 1 or not c.needs_logits)
        self.stats.steps.append(StepStats(
            num_seqs=len(flight.chunks), num_batched_tokens=batched, num_prefill_tokens=prefill,
            num_decode_tokens=batched - prefill, num_preempted=flight.num_preempted,
            schedule_s=(t1 - t0) + (t2 - t1 if ahead is not None else 0.0), forward_s=flight.launch_s + (t3 - t2), postprocess_s=t4 - t3,
        ))
        return outputs

    def generate(self, prompts: Iterable[Sequence[int]], params: SamplingParams | Sequence[SamplingParams] | None = None) -> list[list[int]]:
        """Run prompts to completion; generated ids in input order."""
        prompts = list(prompts)
        per = list(params) if isinstance(params, Sequence) else [params or SamplingParams()] * len(prompts)
        base = next(self._arrivals)
        reqs = [self.add_request(f"gen-{base}-{i}", p, per[i]) for i, p in enumerate(prompts)]
        while self.has_unfinished():
            self.step()
            if self.is_stalled():
                raise RuntimeError("the engine makes no progress: requests wait, nothing runs and nothing could be scheduled")
        return [r.output_ids for r in reqs]

    def is_stalled(self) -> bool:
        """Requests wait, but the last step scheduled nothing, preempted nobody and none is in flight.  Nothing
        changes between steps by itself, so the next step would do the same: whoever owns the
        loop should stop instead of stepping for ever.  (The scheduler's rules exclude this; the
        check is there so that a fault in them ends a run instead of hanging it.)"""
        return (self.has_unfinished() and self._inflight is None and bool(self.stats.steps)
                and self.stats.steps[-1].num_seqs == 0 and self.stats.steps[-1].num_preempted == 0)

    # ------------------------------------------------------------ internals

    def _check_device(self, flight: _InFlight, ahead: _InFlight | None) -> None:
        """The step's ids are on the host, so its kernels have ended: ask the runner whether one of them
        gave up a bounded wait.  If so, nothing the step (or the one launched behind it) computed is
        used: its requests are aborted, no page any of them wrote stays in the prefix index, and the
        error goes to the caller.  The engine itself stays usable."""
        check = getattr(self.runner, "check_device_errors", None)
        if check is None:
            return
        try:
            check()
        except Exception:
            for fl in (flight, ahead):
                for ch in (fl.chunks if fl is not None else []):
                    self._unknown.pop(ch.request.request_id, None)
                    self.scheduler.abort(ch.request.request_id)
            self.manager.reset_prefix_cache()
            raise

    def _sample(self, logits, reqs: list[Request], ahead: int):
        """Ids for ``reqs`` (row order); ``ahead``: tokens of each request that are sampled but not read."""
        if self._by_slot:  # the device knows every request's seed and draw count by its state slot
            return self.sampler.sample_slots_async(logits, [self.manager.state_slot(r.request_id) for r in reqs],
                                                   all_greedy=all(r.params.greedy for r in reqs))
        args = ([r.params for r in reqs], [r.seed for r in reqs], [len(r.output_ids) + ahead for r in reqs])
        if hasattr(self.sampler, "sample_async"):
            return self.sampler.sample_async(logits, *args)
        return _Ready(self.sampler.sample(logits, *args))

    def _run(self, chunks: list[ScheduledChunk], num_preempted: int, token_source=None, token_rows=None, ahead: int = 0) -> _InFlight:
        t0 = time.perf_counter()
        if token_source is None:
            logits = self.runner.execute(chunks)
        else:
            logits = self.runner.execute(chunks, token_source, token_rows)
        for ch in chunks:
            ch.request.num_computed_tokens += ch.num_tokens
            assert self.manager.num_computed_tokens(ch.request.request_id) == ch.request.num_computed_tokens
        sampling = [c.request for c in chunks if c.needs_logits]
        tokens = self._sample(logits, sampling, ahead) if sampling else _Ready([])
        return _InFlight(chunks, sampling, tokens, num_preempted, time.perf_counter() - t0)

    def _launch_scheduled(self) -> _InFlight | None:
        """Ask the scheduler (every id is known to the host) and launch what it chose."""
        sched = self.scheduler.schedule()
        if not sched.chunks:
            self._preempted_for_nothing = len(sched.preempted)  # (a lone request that gave up its own pages)
            return None
        for req in sched.admitted:
            slot = self.manager.state_slot(req.request_id)
            self.runner.start_request(req.request_id, slot)
            if self._by_slot:  # (again after a preemption: the draws made so far are the tokens generated so far)
                self.sampler.bind(slot, req.params, req.seed, len(req.output_ids))
        if sched.copies:
            self.runner.copy_pages(sched.copies)
        return self._run(sched.chunks, len(sched.preempted))

    def _launch_ahead(self, flight: _InFlight) -> _InFlight | None:
        """The decode step that follows ``flight``, launched on the ids it leaves on the device; None
        whenever the scheduler has something to decide first (``Scheduler.schedule_ahead``)."""
        if flight.tokens.device_ids is None:
            return None
        plan = self.scheduler.schedule_ahead(flight.sampling)
        self._unknown.update(plan.unknown)
        if plan.copies:
            self.runner.copy_pages(plan.copies)
        if not plan.chunks:
            return None
        self.steps_ahead += 1
        return self._run(plan.chunks, 0, flight.tokens, plan.token_rows, ahead=1)

    def _resolve(self, flight: _InFlight, tokens: list[int]) -> list[RequestOutput]:
        outputs = []
        for req, tok in zip(flight.sampling, tokens):
            position = self._unknown.pop(req.request_id, None)
            if req.is_finished:
                continue  # ended a step earlier (a stop token, an abort): this token is surplus
            if position is not None and self.manager.has_request(req.request_id):
                self.manager.set_token(req.request_id, position, int(tok))
            outputs.append(self._append_token(req, int(tok)))
        return outputs

    def _append_token(self, req: Request, tok: int) -> RequestOutput:
        req.output_ids.append(tok)
        reason = None
        if tok in req.params.stop_token_ids or (not req.params.ignore_eos and tok in self.eos):
            reason = FinishReason.STOP
        elif len(req.output_ids) >= req.params.max_tokens:
            reason = FinishReason.LENGTH
        if reason is not None:
            self.scheduler.finish(req, reason)
        return RequestOutput(req.request_id, [tok], reason is not None, reason)
