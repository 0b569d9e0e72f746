"""LLMEngine: schedule, run one batched step, sample, update requests, retire the finished.

Names and meanings follow src/dli/engine/engine.py:62-246 (for_model, add_request,
step, generate, abort, has_unfinished, StepStats).  Token ids in, token ids out.
"""

from __future__ import annotations

import itertools
import random
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Collection, Iterable, Protocol, Sequence

from ..sampling import SamplingParams
from .request import FinishReason, Request
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


class LLMEngine:
    def __init__(self, runner: Runner, config: SchedulerConfig | None = None, *, sampler=None,
                 eos_token_ids: Collection[int] = (), seed: int = 0) -> None:
        self.runner = runner
        self.manager = runner.manager
        self.scheduler = Scheduler(config or SchedulerConfig(), self.manager)
        self.sampler = sampler
        self.eos = frozenset(eos_token_ids)
        self._rng = random.Random(seed)
        self._arrivals = itertools.count()
        self.stats = _Counters()

    # ------------------------------------------------------------ construction

    @classmethod
    def for_model(cls, model, *, num_blocks: int | None = None, kv_cache_gb: float | None = None, block_size: int = 16,
                  config: SchedulerConfig | None = None, enable_prefix_caching: bool = True, watermark: float = 0.01,
                  eos_token_ids: Collection[int] = (), seed: int = 0) -> "LLMEngine":
        """An engine around a loaded model.  The cache pool has ``num_blocks`` pages of
        ``block_size`` tokens, or as many as ``kv_cache_gb`` GiB hold (default 1 GiB)."""
        from ..sampling import Sampler
        from .runner import ModelRunner

        config = config or SchedulerConfig()
        if num_blocks is not None and kv_cache_gb is not None:
            raise ValueError("give num_blocks or kv_cache_gb, not both")
        if num_blocks is None:
            num_blocks = ModelRunner.pages_for_budget(model, (kv_cache_gb or 1.0) * 2**30, block_size)
        runner = ModelRunner(model, num_pages=num_blocks, page_size=block_size, max_requests=config.max_num_seqs,
                             enable_prefix_caching=enable_prefix_caching, watermark=watermark)
        return cls(runner, config, sampler=Sampler(model.device), eos_token_ids=eos_token_ids, seed=seed)

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, *, dtype: str = "auto", device: str = "cuda:0", **kwargs) -> "LLMEngine":
        from .runner import load_model

        return cls.for_model(load_model(model_dir, dtype, device), **kwargs)

    # ------------------------------------------------------------ API

    def add_request(self, request_id: str, prompt_ids: Sequence[int], params: SamplingParams | None = None) -> Request:
        """Queue a request.  One that can never fit finishes at once with reason ``capacity``."""
        if not prompt_ids:
            raise ValueError("prompt must be non-empty")
        params = params or SamplingParams()
        seed = params.seed if params.seed is not None else self._rng.getrandbits(63)
        req = Request(request_id, [int(t) for t in prompt_ids], params, next(self._arrivals), seed=seed)
        self.scheduler.add(req)
        return req

    def abort(self, request_id: str) -> bool:
        return self.scheduler.abort(request_id) is not None

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished

    def step(self) -> list[RequestOutput]:
        t0 = time.perf_counter()
        sched = self.scheduler.schedule()
        t1 = time.perf_counter()
        outputs: list[RequestOutput] = []
        if sched.chunks:
            for req in sched.admitted:
                self.runner.start_request(req.request_id, self.manager.state_slot(req.request_id))
            logits = self.runner.execute(sched.chunks)
            t2 = time.perf_counter()
            for ch in sched.chunks:
                ch.request.num_computed_tokens += ch.num_tokens
                assert self.manager.num_computed_tokens(ch.request.request_id) == ch.request.num_computed_tokens
            sampling = [c.request for c in sched.chunks if c.needs_logits]
            tokens = self.sampler.sample(logits, [r.params for r in sampling], [r.seed for r in sampling],
                                         [len(r.output_ids) for r in sampling])
            for req, tok in zip(sampling, tokens):
                outputs.append(self._append_token(req, int(tok)))
        else:
            t2 = t1
        t3 = time.perf_counter()
        prefill = sum(c.num_tokens for c in sched.chunks if c.num_tokens > 1 or not c.needs_logits)
        self.stats.steps.append(StepStats(
            num_seqs=len(sched.chunks), num_batched_tokens=sched.num_batched_tokens, num_prefill_tokens=prefill,
            num_decode_tokens=sched.num_batched_tokens - prefill, num_preempted=len(sched.preempted),
            schedule_s=t1 - t0, forward_s=t2 - t1, postprocess_s=t3 - t2,
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
        return [r.output_ids for r in reqs]

    # ------------------------------------------------------------ internals

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
